"""Chooses the attention kernels of a step.

float32: the CUDA-core kernel for every token (true 32-bit).  bfloat16: tensor-core kernels
where the head size is a multiple of 16 — one launch for the sequences that bring one token
(keys split across CTAs when there are few sequences and long contexts) and one for the longer
portions, which takes the tcgen05 + TMA kernel when head and page size allow it and the
mma.sync kernel otherwise — and the CUDA-core kernel for any other head size.
"""

from __future__ import annotations

import torch

from . import ops

import functools


@functools.lru_cache(maxsize=None)
def sm_count() -> int:
    """SMs of the current CUDA device; without one (host-side tests) the B200's 148."""
    if torch.cuda.is_available():
        return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return 148


def one_wave(ctas_per_sm: int) -> int:
    """CTAs resident at once: the mma.sync decode kernel holds two per SM in its few-sequences shape, the
    TMA-fed decode kernel four at head size 64 and two at head size 128."""
    return sm_count() * ctas_per_sm


MIN_TILES_PER_SPLIT = 2  # key tiles (of 64) a split should at least cover


CLUSTER_SPLITS_MAX = ops.DECODE_TMA_CLUSTER_SPLITS  # splits that the TMA decode kernel merges inside one thread-block cluster
# Splits of the TMA-fed kernel, measured on a B200 with the keys and values not in L2 (head size 64, 8 KV heads;
# us at 1 / 2 / 4 sequences):  8 K keys: 16 splits 15 / 21 / 35, 8 splits 23 / 25 / 27, 64 splits 30 / 36 / 48;
# 32 K keys: 16 splits 27 / 39 / 89, 8 splits 60 / 66 / 68, 32 splits 32 / 48 / 79;  one sequence of 128 K keys: 16
# splits 68, 32 splits 70.  A cluster's merge on the chip beats more splits with a merge kernel at every length a
# model here reaches; a cluster of 16 is worth its narrower placement only while the grid is small (one or two
# sequences' head groups).  (More than 16 splits, merged by a second kernel, remain for callers that ask for them.)
CLUSTER_16_MAX_CTAS_PER_SPLIT = 16


def choose_splits(num_seqs: int, ctas_per_seq: int, max_kv_len: int, wave: int | None = None, fill_last_wave: bool = True) -> int:
    """Key splits for single-token sequences: as many as still fit the GPU in one wave (a second,
    partly filled wave costs more than the extra parallelism brings), none shorter than
    MIN_TILES_PER_SPLIT key tiles (the role of src/dli/model/paged_attention.py:63-74)."""
    wave = one_wave(2) if wave is None else wave
    pairs = max(1, num_seqs * ctas_per_seq)
    tiles = -(-max_kv_len // 64)
    most = max(1, tiles // MIN_TILES_PER_SPLIT)
    if pairs <= wave:
        return max(1, min(wave // pairs, most))
    if not fill_last_wave:
        return 1
    # More CTAs than one wave holds even without splits: a few splits can still fill the last wave
    # (512 CTAs on 296 places leave the second wave 27 % empty; 2,048 fill seven waves to 99 %).  Each
    # split costs merging, so it has to buy three points of occupancy.  (Measured: the mma.sync
    # kernel at head size 128 gains a fifth at 64 sequences; the TMA-fed kernel loses, so it opts out.)
    def score(s: int) -> float:
        ctas = pairs * s
        return ctas / (-(-ctas // wave) * wave) - 0.03 * (s - 1)

    return max(range(1, min(4, most) + 1), key=score)


def decode_splits(num_seqs: int, num_heads: int, nkv: int, head_dim: int, page_size: int, max_kv_len: int) -> int:
    """Key splits of the decode kernel that will serve these sizes."""
    ctas_per_seq = nkv * -(-(num_heads // nkv) // 16)
    tma = ops.decode_tma_supported(head_dim, page_size)
    wave = one_wave(4 if head_dim <= 64 else 2) if tma else one_wave(2)
    splits = choose_splits(num_seqs, ctas_per_seq, max_kv_len, wave, fill_last_wave=not tma)
    if tma and splits > 8:  # a cluster merges its splits on the chip: 16 of them for one or two sequences' head groups, else 8
        pairs = num_seqs * ctas_per_seq
        splits = CLUSTER_SPLITS_MAX if splits >= CLUSTER_SPLITS_MAX and pairs <= CLUSTER_16_MAX_CTAS_PER_SPLIT else 8
    elif tma:
        # The splits of a sequence are a cluster, and clusters of 3 or 6 CTAs run slower than the power of two below
        # them.  Measured in replayed graphs (us a launch, splits 2 / 3 / 4): 24 sequences at head size 64 and 2 K keys
        # 21.8 / 31.4 / 28.7, at 16 K keys 139 / 161 / 136; 12 sequences at head size 128 and 2 K keys 21.9 / 34.5 /
        # 29.5; 12 sequences at head size 64 with 4 / 6 splits 13.5 / 20.1.
        splits = 1 << (splits.bit_length() - 1)
    return splits


def paged_attention(out: torch.Tensor, qkv: torch.Tensor, cache, batch, num_heads: int, scale: float, window: int | None,
                    splits: int | None = None) -> None:
    """Attention of every token of the step over its sequence's pages.  ``splits``: key runs per single-token
    sequence, if the caller fixed them (a recorded graph); otherwise chosen from this step's shape."""
    group = batch.group(cache.group)
    _, nkv, _, d = cache.k.shape
    if out.dtype != torch.bfloat16 or not ops.mma_head_dim_supported(d):
        ops.paged_attention_simt(out, qkv, cache.k, cache.v, group.block_tables, batch.seq_of_token, batch.positions,
                                 num_heads, scale, window)
        return
    singles, total = batch.num_single, batch.num_seqs
    if singles:
        tma = ops.decode_tma_supported(d, cache.page_size)
        splits = splits or decode_splits(singles, num_heads, nkv, d, cache.page_size, batch.max_kv_len_single)
        scratch = None
        if splits > 1:
            rows = singles * num_heads
            scratch = (torch.empty(rows * splits * d, dtype=torch.float32, device=out.device),
                       torch.empty(rows * splits * 2, dtype=torch.float32, device=out.device))
        kernel = ops.paged_decode_tma if tma else ops.paged_attention_mma
        args = (out, qkv, cache.k, cache.v, group.block_tables, batch.q_start, batch.kv_len, 0, singles) + (() if tma else (1,))
        kernel(*args, 0, num_heads, scale, window, splits, scratch, *((batch.max_kv_len_single,) if tma else ()))
    if total > singles and ops.prefill_tc_supported(d, cache.page_size):
        ops.paged_prefill_tc(out, qkv, cache.k, cache.v, group.block_tables, batch.q_start, batch.kv_len, singles, total - singles,
                             batch.max_q_len, num_heads, scale, window)
    elif total > singles:
        ops.paged_attention_mma(out, qkv, cache.k, cache.v, group.block_tables, batch.q_start, batch.kv_len, singles,
                                total - singles, batch.max_q_len, singles, num_heads, scale, window)
