"""The host-side choice of key splits for single-token sequences (kernels/attention.py): no GPU needed."""

from dli_b200.kernels.attention import CLUSTER_SPLITS_MAX, decode_splits


def splits(seqs, ctx, heads=32, nkv=8, d=64, page=16):
    return decode_splits(seqs, heads, nkv, d, page, ctx)


def test_short_contexts_are_not_cut_below_two_key_tiles():
    assert splits(1, 100) == 1
    assert splits(1, 300) == 2
    assert splits(64, 2048) == 1  # the grid is full without splits


def test_few_sequences_merge_in_a_cluster():
    assert [splits(1, c) for c in (2048, 8192, 16384)] == [CLUSTER_SPLITS_MAX] * 3
    assert [splits(2, c) for c in (2048, 8192, 65536)] == [CLUSTER_SPLITS_MAX] * 3
    assert [splits(4, c) for c in (2048, 8192, 65536)] == [8] * 3  # a cluster of 16 only while the grid is small
    assert splits(8, 2048) == 8
    assert splits(16, 8192) == 4  # one wave of CTAs


def test_long_sequences_stay_with_a_cluster():
    assert splits(1, 49152) == CLUSTER_SPLITS_MAX and splits(1, 131072) == CLUSTER_SPLITS_MAX
    assert splits(2, 65536) == CLUSTER_SPLITS_MAX and splits(4, 131072) == 8
    assert splits(1, 65536, heads=24, d=128) == CLUSTER_SPLITS_MAX


def test_a_cluster_of_splits_is_a_power_of_two():
    """One wave of CTAs would allow 3 splits at 24 sequences and 6 at 12; clusters of those sizes are slower than
    the power of two below."""
    assert splits(24, 2048) == 2 and splits(20, 8192) == 2
    assert splits(12, 2048) == 4 and splits(10, 8192) == 4
    assert splits(12, 8192, heads=24, d=128) == 2
    for seqs in range(1, 80):
        for ctx in (256, 2048, 16384):
            s = splits(seqs, ctx)
            assert s & (s - 1) == 0
