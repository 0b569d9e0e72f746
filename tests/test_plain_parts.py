"""Each function of the plain implementation against an even plainer restatement (loops, known
answers, invariants), so that the oracle the GPU tests lean on is itself anchored.  No GPU."""

import math

import numpy as np
import pytest
import torch

from tests.plain import llama_plain as plain


def test_philox_known_answers():
    """Philox-4x32-10 test vectors as published with the generator (zeros, all ones, digits of pi)."""
    assert plain.philox4x32((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    ones = 0xFFFFFFFF
    assert plain.philox4x32((ones,) * 4, (ones, ones)) == (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)
    assert plain.philox4x32((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0)) == (
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)


def test_uniform_numbers_depend_on_seed_and_draw_only_and_fill_the_interval():
    u = np.array([plain.uniform_for_draw(7, i) for i in range(4000)])
    assert (u >= 0).all() and (u < 1).all() and abs(u.mean() - 0.5) < 0.02 and abs((u < 0.1).mean() - 0.1) < 0.02
    assert plain.uniform_for_draw(7, 5) == u[5] != plain.uniform_for_draw(8, 5)
    assert plain.uniform_for_draw(2**40 + 3, 2**33) != plain.uniform_for_draw(3, 2**33)  # the high words count


def test_rms_norm_by_hand():
    x = np.array([[3.0, -4.0, 0.0, 0.0]], dtype=np.float32)
    w = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)
    want = w * x / math.sqrt((9 + 16) / 4 + 1e-3)
    np.testing.assert_allclose(plain.rms_norm(x, w, 1e-3), want, rtol=1e-6)


def test_rope_is_a_rotation_that_depends_on_the_distance():
    d, n = 16, 40
    c = {"head_dim": d, "theta": 10000.0, "rope_type": "default"}
    inv = plain.inverse_frequencies(c)
    np.testing.assert_allclose(inv, [10000.0 ** (-2 * j / d) for j in range(d // 2)], rtol=1e-6)
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 1, d)).astype(np.float32), rng.standard_normal((1, 1, d)).astype(np.float32)

    def at(x, pos):
        cos, sin = plain.rope_cos_sin(inv, np.array([pos]))
        return plain.apply_rope(x, cos, sin)

    np.testing.assert_allclose(at(q, 0), q, atol=1e-7)  # position 0 leaves the vector alone
    np.testing.assert_allclose(np.linalg.norm(at(q, 17)), np.linalg.norm(q), rtol=1e-6)
    dots = [float((at(q, m) * at(k, m - 5)).sum()) for m in (5, 9, n)]
    np.testing.assert_allclose(dots, dots[0], rtol=1e-4, atol=1e-5)  # the score depends on m - n alone
    # element j pairs with element j + d/2 (rotate-half), not with its neighbour
    e0 = np.zeros((1, 1, d), dtype=np.float32)
    e0[..., 0] = 1
    r = at(e0, 1)[0, 0]
    assert abs(r[0] - math.cos(1.0)) < 1e-6 and abs(r[d // 2] - math.sin(1.0)) < 1e-6 and abs(r[1]) < 1e-7


@pytest.mark.parametrize("window", [None, 3])
def test_causal_attention_by_loops(window):
    rng = np.random.default_rng(1)
    heads, kvh, n, d = 4, 2, 7, 8
    q = rng.standard_normal((heads, n, d)).astype(np.float32)
    k = rng.standard_normal((kvh, n, d)).astype(np.float32)
    v = rng.standard_normal((kvh, n, d)).astype(np.float32)
    want = np.zeros((heads, n, d))
    for h in range(heads):
        g = h // (heads // kvh)
        for i in range(n):
            keys = [j for j in range(i + 1) if window is None or i - j < window]
            s = np.array([q[h, i].astype(np.float64) @ k[g, j] / math.sqrt(d) for j in keys])
            p = np.exp(s - s.max())
            p /= p.sum()
            want[h, i] = sum(pj * v[g, j] for pj, j in zip(p, keys))
    np.testing.assert_allclose(plain.causal_attention(q, k, v, window), want, atol=1e-5)


def test_swiglu_by_hand():
    w = {"m.gate_proj.weight": np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=np.float32),
         "m.up_proj.weight": np.array([[2.0, 0.0], [0.0, -1.0], [0.5, 0.5]], dtype=np.float32),
         "m.down_proj.weight": np.array([[1.0, 1.0, 1.0], [0.0, 2.0, 0.0]], dtype=np.float32)}
    x = np.array([[1.0, -2.0]], dtype=np.float32)
    gate, up = np.array([1.0, -2.0, -1.0]), np.array([2.0, 2.0, -0.5])
    act = gate / (1 + np.exp(-gate)) * up
    np.testing.assert_allclose(plain.swiglu_mlp(x, w, "m."), [[act.sum(), 2 * act[1]]], rtol=1e-6)


def test_round_to_bfloat16_is_ties_to_even():
    x = torch.randn(10000).numpy() * np.float32(3.0)
    special = np.array([1.0 + 2**-8, 1.0 + 3 * 2**-8, 1.0 + 2**-9, -1.0 - 2**-8, 0.0, 65280.0], dtype=np.float32)  # two exact ties
    x = np.concatenate([x, special]).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(plain.round_to_bfloat16(x), want)
    assert plain.round_to_bfloat16(np.float32([1.0 + 2**-8]))[0] == 1.0  # the tie goes to the even mantissa
    assert plain.round_to_bfloat16(np.float32([1.0 + 3 * 2**-8]))[0] == np.float32(1.0 + 2**-6)


def test_filtered_probabilities_rules():
    logits = np.log(np.array([0.4, 0.3, 0.2, 0.1]))
    np.testing.assert_allclose(plain.filtered_probabilities(logits, 1.0), [0.4, 0.3, 0.2, 0.1], rtol=1e-12)
    np.testing.assert_allclose(plain.filtered_probabilities(logits, 1.0, top_k=2), [4 / 7, 3 / 7, 0, 0], rtol=1e-12)
    # top_p: a token goes when the tokens more likely than it already hold top_p of the mass
    np.testing.assert_allclose(plain.filtered_probabilities(logits, 1.0, top_p=0.7), [4 / 7, 3 / 7, 0, 0], rtol=1e-12)
    np.testing.assert_allclose(plain.filtered_probabilities(logits, 1.0, top_p=0.71), [4 / 9, 3 / 9, 2 / 9, 0], rtol=1e-12)
    np.testing.assert_allclose(plain.filtered_probabilities(logits, 1.0, top_p=1e-9), [1, 0, 0, 0])  # the top token always stays
    sharp = plain.filtered_probabilities(logits, 0.5)
    np.testing.assert_allclose(sharp, np.array([0.16, 0.09, 0.04, 0.01]) / 0.30, rtol=1e-12)
    # token order is kept whatever the order of the logits
    np.testing.assert_allclose(plain.filtered_probabilities(logits[::-1].copy(), 1.0, top_k=2), [0, 0, 3 / 7, 4 / 7], rtol=1e-12)


def test_sample_token_follows_the_distribution_and_greedy_takes_the_lowest_id():
    logits = np.log(np.array([0.5, 0.25, 0.125, 0.125]))
    draws = np.array([plain.sample_token(logits, 1.0, -1, 1.0, 11, i) for i in range(8000)])
    freq = np.bincount(draws, minlength=4) / draws.size
    np.testing.assert_allclose(freq, [0.5, 0.25, 0.125, 0.125], atol=0.02)
    assert plain.sample_token(np.array([1.0, 3.0, 3.0, 0.0]), 0.0, -1, 1.0, 0, 0) == 1
    assert plain.sample_token(np.array([1.0, 3.0, 3.0, 0.0]), 0.9, 1, 1.0, 0, 0) == 1  # top_k == 1 is greedy
    assert all(plain.sample_token(logits, 1.0, 2, 1.0, 3, i) in (0, 1) for i in range(200))
    assert [plain.sample_token(logits, 1.0, -1, 1.0, 5, i) for i in range(20)] == [plain.sample_token(logits, 1.0, -1, 1.0, 5, i) for i in range(20)]


def test_read_config_defaults_follow_the_reference():
    c = plain.read_config({"num_attention_heads": 4, "hidden_size": 32, "vocab_size": 10, "intermediate_size": 8,
                           "num_hidden_layers": 1, "rms_norm_eps": 1e-5})
    assert c["kv_heads"] == 4 and c["head_dim"] == 8 and c["theta"] == 10000.0 and c["rope_type"] == "default" and not c["tied"]
    with pytest.raises(KeyError):
        plain.read_config({"num_attention_heads": 4, "hidden_size": 32, "vocab_size": 10, "intermediate_size": 8, "num_hidden_layers": 1})
