"""Each CUDA kernel alone against a plain float64/float32 restatement, at sizes other than
the engine's tiny and benchmark models; inputs are made so that a wrong key, a page edge or a
window edge shows."""

import math

import numpy as np
import pytest
import torch

from dli_b200.kernels import ops
from dli_b200.kernels.attention import choose_splits
from tests.plain import llama_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------ elementwise


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    table = rnd(300, 80, dtype=dtype)
    ids = torch.tensor([0, 299, 7, 7, 150], dtype=torch.int32, device=DEV)
    h = torch.empty(5, 80, dtype=torch.float32, device=DEV)
    ops.embedding(h, table, ids)
    assert torch.equal(h, table.float()[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [80, 2064, 5000])
def test_add_rmsnorm(dtype, H):
    h = rnd(6, H, seed=1)
    delta = rnd(6, H, dtype=dtype, seed=2)
    w = 1 + 0.1 * rnd(H, seed=3)
    eps = 3e-6
    want_h = h.double() + delta.double()
    want_y = plain.rms_norm(want_h.cpu().numpy(), w.double().cpu().numpy(), eps)
    y = torch.empty(6, H, dtype=dtype, device=DEV)
    h1 = h.clone()
    ops.add_rmsnorm(y, h1, delta, w, eps)
    np.testing.assert_allclose(h1.cpu().numpy(), want_h.float().cpu().numpy(), rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(y.float().cpu().numpy(), want_y, atol=tol(dtype, 4))
    # rows so small that eps decides the scale
    hs = h * 1e-3
    ops.add_rmsnorm(y, hs.clone(), None, w, 1e-5)
    np.testing.assert_allclose(y.float().cpu().numpy(), plain.rms_norm(hs.double().cpu().numpy(), w.double().cpu().numpy(), 1e-5), atol=tol(dtype, 4))
    # without delta the stream is left alone
    h2 = h.clone()
    ops.add_rmsnorm(y, h2, None, w, eps)
    assert torch.equal(h2, h)
    np.testing.assert_allclose(y.float().cpu().numpy(), plain.rms_norm(h.double().cpu().numpy(), w.double().cpu().numpy(), eps), atol=tol(dtype, 4))
    # selected rows: only those are read, nothing is written back
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    y3 = torch.empty(3, H, dtype=dtype, device=DEV)
    h3 = h.clone()
    ops.add_rmsnorm(y3, h3, delta, w, eps, rows)
    assert torch.equal(h3, h)
    np.testing.assert_allclose(y3.float().cpu().numpy(), want_y[[4, 0, 4]], atol=tol(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rot", [48, 32, 0])
def test_rotary_store(dtype, rot):
    nh, nkv, d, page, pages, n = 5, 1, 48, 8, 6, 7
    qkv = rnd(n, (nh + 2 * nkv) * d, dtype=dtype, seed=4)
    positions = torch.tensor([0, 1, 63, 64, 4095, 100000, 17], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 8, 47, 0, 16, -1, 23], dtype=torch.int32, device=DEV)
    kp = torch.full((pages, nkv, page, d), 9.0, dtype=dtype, device=DEV)
    vp = torch.full((pages, nkv, page, d), 9.0, dtype=dtype, device=DEV)
    inv = None
    x = qkv.double().cpu().numpy().reshape(n, nh + 2 * nkv, d)
    want = x.copy()
    if rot:
        c = {"head_dim": rot, "theta": 500000.0, "rope_type": "llama3", "factor": 8.0, "low": 1.0, "high": 4.0, "old_ctx": 64}
        inv_np = plain.inverse_frequencies(c)
        inv = torch.from_numpy(inv_np).to(DEV)
        cos, sin = plain.rope_cos_sin(inv_np, positions.cpu().numpy())
        heads = x[:, : nh + nkv, :rot].transpose(1, 0, 2)
        want[:, : nh + nkv, :rot] = plain.apply_rope(heads, cos.astype(np.float64), sin.astype(np.float64)).transpose(1, 0, 2)
    got = qkv.clone()
    ops.rotary_store(got, positions, inv, slots, kp, vp, nh, nkv, d, rot, page)
    g = got.double().cpu().numpy().reshape(n, nh + 2 * nkv, d)
    np.testing.assert_allclose(g[:, :nh], want[:, :nh], atol=tol(dtype, 4))
    np.testing.assert_array_equal(g[:, nh:], x[:, nh:])  # k and v columns of qkv are not touched
    kflat = kp.double().cpu().numpy().transpose(0, 2, 1, 3).reshape(pages * page, nkv, d)
    vflat = vp.double().cpu().numpy().transpose(0, 2, 1, 3).reshape(pages * page, nkv, d)
    written = set()
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        written.add(s)
        np.testing.assert_allclose(kflat[s], want[t, nh : nh + nkv], atol=tol(dtype, 4))
        np.testing.assert_array_equal(vflat[s], x[t, nh + nkv :])
    untouched = [s for s in range(pages * page) if s not in written]
    assert (kflat[untouched] == 9.0).all() and (vflat[untouched] == 9.0).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    gu = rnd(7, 400, dtype=dtype, seed=5, scale=3.0)
    out = torch.empty(7, 200, dtype=dtype, device=DEV)
    ops.silu_mul(out, gu)
    g = gu.double().cpu().numpy()
    np.testing.assert_allclose(out.float().cpu().numpy(), plain.silu(g[:, :200]) * g[:, 200:], atol=tol(dtype, 10))


# ------------------------------------------------------------------ attention


def attention_case(nh, nkv, d, page, seqs, dtype, seed=0, sharp=None, ramp=0.0):
    """seqs: [(start, q_len)].  Builds pools with shuffled pages, tables whose unused entries
    point at a poisoned page (NaN: a stray read shows without faulting), qkv rows, and the plain
    result.  sharp = (seq, token, key): that query and key are scaled so the score stands out.
    ramp: every query gets a component along one direction and key u one of ramp * u along it, so
    scores grow with the key's position and a row's maximum rises from tile to tile."""
    rng = np.random.default_rng(seed)
    kv_lens = [s + q for s, q in seqs]
    blocks = [-(-k // page) for k in kv_lens]
    pages = sum(blocks) + 1
    poison = pages - 1
    perm = rng.permutation(pages - 1)
    tables = np.full((len(seqs), max(blocks) + 2), poison, dtype=np.int32)
    at = 0
    for i, b in enumerate(blocks):
        tables[i, :b] = perm[at : at + b]
        at += b
    K = [rng.standard_normal((k, nkv, d)) for k in kv_lens]
    V = [rng.standard_normal((k, nkv, d)) for k in kv_lens]
    Q = [rng.standard_normal((q, nh, d)) for _, q in seqs]
    if sharp is not None:
        si, ti, ki = sharp
        direction = rng.standard_normal(d)
        direction /= np.linalg.norm(direction)
        Q[si][ti] = direction * 6.0 * math.sqrt(math.sqrt(d))
        K[si][ki] = direction * 6.0 * math.sqrt(math.sqrt(d))
    if ramp:
        direction = rng.standard_normal(d)
        direction /= np.linalg.norm(direction)
        for i in range(len(seqs)):
            Q[i] = 0.3 * Q[i] + direction * math.sqrt(d)
            K[i] = 0.3 * K[i] + direction[None, None, :] * (ramp * np.arange(kv_lens[i]))[:, None, None]
    tt = torch.float32 if dtype == torch.float32 else torch.bfloat16
    cast = lambda a: torch.from_numpy(a).to(tt)
    K, V, Q = [[cast(a) for a in L] for L in (K, V, Q)]
    kp = torch.full((pages, nkv, page, d), float("nan"), dtype=tt)
    vp = torch.full((pages, nkv, page, d), float("nan"), dtype=tt)
    for i, klen in enumerate(kv_lens):
        for pos in range(klen):
            pg = tables[i, pos // page]
            kp[pg, :, pos % page] = K[i][pos]
            vp[pg, :, pos % page] = V[i][pos]
    # rows of a half-used page beyond the sequence hold finite junk, as a reused page would
    for i, klen in enumerate(kv_lens):
        if klen % page:
            pg = tables[i, klen // page]
            kp[pg, :, klen % page :] = 1e4
            vp[pg, :, klen % page :] = 1e4
    n = sum(q for _, q in seqs)
    qkv = torch.zeros(n, (nh + 2 * nkv) * d, dtype=tt)
    qkv[:, : nh * d] = torch.cat([q.reshape(q.shape[0], nh * d) for q in Q])
    q_start = np.cumsum([0] + [q for _, q in seqs]).astype(np.int32)
    seq_of_token = np.concatenate([np.full(q, i, dtype=np.int32) for i, (_, q) in enumerate(seqs)])
    positions = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in seqs])
    dev = lambda a: (a if isinstance(a, torch.Tensor) else torch.from_numpy(a)).to(DEV).contiguous()
    t = dict(qkv=dev(qkv), kp=dev(kp), vp=dev(vp), tables=dev(tables), q_start=dev(q_start), kv_len=dev(np.array(kv_lens, dtype=np.int32)),
             seq_of_token=dev(seq_of_token), positions=dev(positions), n=n, Q=Q, K=K, V=V)
    return t


def plain_attention(t, seqs, nh, window):
    outs = []
    for i, (start, qlen) in enumerate(seqs):
        klen = start + qlen
        # run the whole sequence through the plain causal attention, keep the last q_len rows
        qfull = np.zeros((nh, klen, t["Q"][i].shape[-1]))
        qfull[:, start:] = t["Q"][i].double().numpy().transpose(1, 0, 2)
        o = plain.causal_attention(qfull, t["K"][i].double().numpy().transpose(1, 0, 2), t["V"][i].double().numpy().transpose(1, 0, 2), window)
        outs.append(o[:, start:].transpose(1, 0, 2).reshape(qlen, -1))
    return np.concatenate(outs)


SHAPES = [(4, 2, 16, 4), (3, 1, 32, 16), (5, 5, 48, 8), (8, 2, 64, 16), (6, 1, 128, 32), (2, 2, 256, 16), (7, 7, 80, 5)]
MIX = [(0, 1), (199, 1), (63, 1), (0, 37), (40, 2), (64, 64), (3, 130), (255, 1), (16, 17)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,page", SHAPES)
@pytest.mark.parametrize("window", [None, 70, 5])
def test_paged_attention_simt(dtype, nh, nkv, d, page, window):
    t = attention_case(nh, nkv, d, page, MIX, dtype, seed=nh)
    out = torch.empty(t["n"], nh * d, dtype=dtype, device=DEV)
    ops.paged_attention_simt(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["seq_of_token"], t["positions"], nh, d**-0.5, window)
    want = plain_attention(t, MIX, nh, window)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(dtype, 2))


def run_mma(t, seqs, nh, d, window, splits=1):
    """Single-token sequences first (the engine's order is the caller's duty here)."""
    singles = sum(1 for _, q in seqs if q == 1)
    assert all(q == 1 for _, q in seqs[:singles]) and all(q > 1 for _, q in seqs[singles:])
    out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    if singles:
        scratch = None
        if splits > 1:
            scratch = (torch.full((singles * nh * splits * d,), float("nan"), device=DEV), torch.full((singles * nh * splits * 2,), float("nan"), device=DEV))
        ops.paged_attention_mma(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, singles, 1, 0, nh, d**-0.5, window, splits, scratch)
    if len(seqs) > singles:
        ops.paged_attention_mma(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], singles, len(seqs) - singles,
                                max(q for _, q in seqs), singles, nh, d**-0.5, window)
    return out


ORDERED = sorted(MIX, key=lambda sq: sq[1] != 1)


@pytest.mark.parametrize("nh,nkv,d,page", [s for s in SHAPES if s[2] % 16 == 0] + [(128, 1, 32, 16), (70, 1, 16, 16)])
@pytest.mark.parametrize("window", [None, 70, 5])
@pytest.mark.parametrize("splits", [1, 3])
def test_paged_attention_mma(nh, nkv, d, page, window, splits):
    t = attention_case(nh, nkv, d, page, ORDERED, torch.bfloat16, seed=nh + d)
    out = run_mma(t, ORDERED, nh, d, window, splits)
    want = plain_attention(t, ORDERED, nh, window)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2))


PREFILL_MIX = [(0, 37), (40, 2), (64, 64), (3, 130), (255, 300), (16, 17), (700, 129), (0, 128)]


@pytest.mark.parametrize("nh,nkv,page", [(8, 2, 16), (3, 1, 8), (5, 5, 32), (4, 4, 128), (32, 8, 64), (130, 1, 16)])
@pytest.mark.parametrize("window", [None, 70, 200])
def test_paged_prefill_tc(nh, nkv, page, window):
    """The tcgen05 + TMA prefill kernels (one and two query tiles per CTA): portions that start anywhere,
    cross tile and page edges, with GQA groups from 1 to 130 heads per KV head."""
    d = 64
    t = attention_case(nh, nkv, d, page, PREFILL_MIX, torch.bfloat16, seed=nh + page)
    want = plain_attention(t, PREFILL_MIX, nh, window)
    for tiles in (1, 2, 0):
        out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.paged_prefill_tc(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(PREFILL_MIX),
                             max(q for _, q in PREFILL_MIX), nh, d**-0.5, window, tiles)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2), err_msg=f"{tiles} query tiles")
    assert ops.paged_prefill_tc_error() == 0


DECODE_TMA_CASES = [(64, nh, nkv, page, window, splits)
                    for nh, nkv, page in [(8, 2, 16), (3, 1, 8), (5, 5, 32), (32, 8, 64), (40, 1, 16)] for window in (None, 70) for splits in (1, 3, 8)]
DECODE_TMA_CASES += [(64, 8, 2, 16, None, 11), (128, 24, 8, 16, None, 1), (128, 24, 8, 16, 70, 8), (128, 3, 1, 8, None, 3), (128, 3, 1, 8, 70, 1),
                     (128, 20, 1, 32, None, 11), (128, 4, 4, 128, None, 8)]


@pytest.mark.parametrize("d,nh,nkv,page,window,splits", DECODE_TMA_CASES)
def test_paged_decode_tma(nh, nkv, page, window, splits, d):
    """The TMA-fed decode kernel at both head sizes: contexts from 1 to 1500 keys, ends on and off tile
    and page edges; splits merged inside a cluster (up to 8) and by the merge kernel (11)."""
    seqs = [(0, 1), (15, 1), (16, 1), (199, 1), (63, 1), (255, 1), (1499, 1), (700, 1)]
    t = attention_case(nh, nkv, d, page, seqs, torch.bfloat16, seed=nh + page)
    out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    scratch = None
    if splits > 1:
        scratch = (torch.full((len(seqs) * nh * splits * d,), float("nan"), device=DEV), torch.full((len(seqs) * nh * splits * 2,), float("nan"), device=DEV))
    ops.paged_decode_tma(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(seqs), 0, nh, d**-0.5, window, splits, scratch)
    want = plain_attention(t, seqs, nh, window)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2))
    assert ops.paged_prefill_tc_error() == 0


def plain_decode_rows(t, seqs, nh, window=None):
    """Attention of each sequence's one query over all its keys (the last ``window`` of them), in float64, row by row
    (the whole-sequence restatement above would build a square of scores per head, which thousands of keys make too large)."""
    outs = []
    for i in range(len(seqs)):
        q = t["Q"][i].double().numpy()[0]  # [nh, d]
        K, V = t["K"][i].double().numpy(), t["V"][i].double().numpy()  # [keys, nkv, d]
        if window:
            K, V = K[-window:], V[-window:]
        fan = nh // K.shape[1]
        row = []
        for h in range(nh):
            sc = K[:, h // fan] @ q[h] / math.sqrt(q.shape[-1])
            w = np.exp(sc - sc.max())
            row.append((w / w.sum()) @ V[:, h // fan])
        outs.append(np.concatenate(row))
    return np.stack(outs)


@pytest.mark.parametrize("d,nh,nkv,page,splits,lens", [
    (64, 32, 8, 16, 16, [2048, 2049, 2500, 3071]),  # one cluster of 16 CTAs merges the splits (what one sequence at 2 K..3 K keys gets)
    (64, 32, 8, 16, 24, [4096, 5003]),  # beyond a cluster: partial results in scratch, merged by the merge kernel
    (64, 32, 8, 16, 32, [4100, 6001, 33]),
    (64, 3, 1, 8, 16, [2300]),
    (128, 24, 8, 16, 16, [2048, 3000]),
    (128, 24, 8, 16, 32, [4200, 8100]),
])
def test_paged_decode_tma_many_splits_over_long_contexts(d, nh, nkv, page, splits, lens):
    """The split counts the engine picks for few sequences with thousands of keys: 16 (merged on the chip by a
    cluster of the non-portable size 16) and 24 / 32 (merge kernel), contexts that end on and off tile edges,
    one sequence far shorter than a split's share."""
    seqs = [(n - 1, 1) for n in lens]
    t = attention_case(nh, nkv, d, page, seqs, torch.bfloat16, seed=splits + len(lens), sharp=(0, 0, lens[0] // 3))
    out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    scratch = (torch.full((len(seqs) * nh * splits * d,), float("nan"), device=DEV), torch.full((len(seqs) * nh * splits * 2,), float("nan"), device=DEV))
    ops.paged_decode_tma(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(seqs), 0, nh, d**-0.5, None, splits, scratch)
    np.testing.assert_allclose(out.float().cpu().numpy(), plain_decode_rows(t, seqs, nh), atol=tol(torch.bfloat16, 2))
    assert ops.paged_prefill_tc_error() == 0


@pytest.mark.parametrize("nh,nkv,page,window,keys", [(32, 8, 16, None, 8300), (32, 8, 16, 5000, 9001), (3, 1, 8, None, 8200), (8, 8, 64, None, 16400)])
def test_paged_decode_tma_with_eight_warps_a_cta(nh, nkv, page, window, keys):
    """One long sequence at head size 64: told the length, the launcher gives a CTA eight warps instead of four (the
    grid is smaller than the GPU and every warp still has four tiles or more).  The result is that of four warps and
    of the plain softmax."""
    d, splits = 64, 16
    seqs = [(keys - 1, 1)]
    t = attention_case(nh, nkv, d, page, seqs, torch.bfloat16, seed=keys % 97, sharp=(0, 0, keys // 3))
    want = plain_decode_rows(t, seqs, nh, window)
    outs = []
    for hint in (0, keys):
        out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        scratch = (torch.full((nh * splits * d,), float("nan"), device=DEV), torch.full((nh * splits * 2,), float("nan"), device=DEV))
        ops.paged_decode_tma(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, 1, 0, nh, d**-0.5, window, splits, scratch, hint)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2), err_msg=f"length hint {hint}")
        outs.append(out.float().cpu().numpy())
    np.testing.assert_allclose(outs[0], outs[1], atol=tol(torch.bfloat16, 1))
    assert ops.paged_prefill_tc_error() == 0


@pytest.mark.parametrize("ramp", [0.02, 0.3])
@pytest.mark.parametrize("d", [64, 128])
def test_decode_tma_when_row_maxima_keep_rising(ramp, d):
    """Scores that grow with the key's position: the decode kernel's reference maximum stays where it is over many
    tiles (0.02: a sixteenth of a power of two per 16-key tile, far below its step of 2^8) or moves at every tile
    (0.3), with one, a few and sixteen splits."""
    nh, nkv, page = 8, 2, 16
    seqs = [(699, 1), (2999, 1), (15, 1)]
    t = attention_case(nh, nkv, d, page, seqs, torch.bfloat16, seed=6, ramp=ramp)
    want = plain_decode_rows(t, seqs, nh)
    for splits in (1, 3, 16):
        out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        scratch = (torch.full((len(seqs) * nh * splits * d,), float("nan"), device=DEV), torch.full((len(seqs) * nh * splits * 2,), float("nan"), device=DEV))
        ops.paged_decode_tma(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(seqs), 0, nh, d**-0.5, None, splits, scratch if splits > 1 else None)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2), err_msg=f"{splits} splits")
    assert ops.paged_prefill_tc_error() == 0


@pytest.mark.parametrize("nh,nkv,page,window", [(6, 2, 16, None), (3, 1, 8, 70), (4, 4, 128, None), (24, 8, 32, 200), (9, 1, 16, None)])
def test_paged_prefill_tc_head_size_128(nh, nkv, page, window):
    """Head size 128 goes to the kernel with a thread per row: two 128-byte slabs per row of keys and values."""
    d = 128
    t = attention_case(nh, nkv, d, page, PREFILL_MIX, torch.bfloat16, seed=nh + page)
    want = plain_attention(t, PREFILL_MIX, nh, window)
    out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_prefill_tc(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(PREFILL_MIX),
                         max(q for _, q in PREFILL_MIX), nh, d**-0.5, window)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2))
    assert ops.paged_prefill_tc_error() == 0


@pytest.mark.parametrize("ramp", [0.02, 0.3])
def test_prefill_tc_when_row_maxima_keep_rising(ramp):
    """Scores that grow with the key's position: the row maxima rise by a little (0.02: about four powers
    of two per tile, below the kernel's step for rescaling its accumulated output) or by a lot (0.3: about
    55 per tile, a rescaling at every tile)."""
    nh, nkv, d, page = 8, 2, 64, 16
    seqs = [(0, 700), (300, 260), (1000, 3)]
    t = attention_case(nh, nkv, d, page, seqs, torch.bfloat16, seed=5, ramp=ramp)
    want = plain_attention(t, seqs, nh, None)
    for tiles in (1, 2):
        out = torch.full((t["n"], nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.paged_prefill_tc(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(seqs), max(q for _, q in seqs), nh, d**-0.5, None, tiles)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=tol(torch.bfloat16, 2), err_msg=f"{tiles} query tiles")
    assert ops.paged_prefill_tc_error() == 0


def test_prefill_tc_refuses_other_sizes():
    t = attention_case(2, 1, 32, 16, [(0, 4)], torch.bfloat16)
    out = torch.empty((4, 64), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.KernelError, match="head_dim"):
        ops.paged_prefill_tc(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, 1, 4, 2, 1.0)
    assert not ops.prefill_tc_supported(64, 4) and not ops.prefill_tc_supported(64, 48)


def test_mma_rejects_other_head_sizes():
    t = attention_case(2, 1, 24, 8, [(0, 4)], torch.bfloat16)
    with pytest.raises(ops.KernelError, match="multiple of 16"):
        run_mma(t, [(0, 4)], 2, 24, None)


@pytest.mark.parametrize("kernel", ["simt-f32", "simt-bf16", "mma", "tc"])
@pytest.mark.parametrize("where", ["far_key", "page_first", "page_last", "tile_edge_63", "tile_edge_64", "window_inside", "window_outside", "self"])
def test_one_key_stands_out(kernel, where):
    """The query of one token matches one key so strongly that the output is that key's value.
    The key sits where an indexing fault would hide among random data: far back among hundreds,
    on both sides of a page edge and of a 64-key tile edge, and on both sides of a window edge."""
    nh, nkv, d, page = 4, 2, 64, 16
    start, qlen = 600, 40
    token = 25
    pos = start + token
    window = None
    key = {"far_key": 3, "page_first": 16 * 20, "page_last": 16 * 20 - 1, "tile_edge_63": 64 * 5 - 1, "tile_edge_64": 64 * 5, "self": pos}.get(where)
    if where.startswith("window"):
        window = 100
        key = pos - window + 1 if where == "window_inside" else pos - window
    dtype = torch.float32 if kernel == "simt-f32" else torch.bfloat16
    seqs = [(12, 1), (start, qlen)]
    t = attention_case(nh, nkv, d, page, seqs, dtype, seed=11, sharp=(1, token, key))
    if kernel == "mma":
        out = run_mma(t, seqs, nh, d, window)
    elif kernel == "tc":
        out = run_mma(t, seqs[:1], nh, d, window)  # the single-token sequence
        ops.paged_prefill_tc(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 1, 1, qlen, nh, d**-0.5, window)
    else:
        out = torch.empty(t["n"], nh * d, dtype=dtype, device=DEV)
        ops.paged_attention_simt(out, t["qkv"], t["kp"], t["vp"], t["tables"], t["seq_of_token"], t["positions"], nh, d**-0.5, window)
    want = plain_attention(t, seqs, nh, window)
    got = out.float().cpu().numpy()
    np.testing.assert_allclose(got, want, atol=tol(dtype, 4))
    row = got[1 + token].reshape(nh, d)
    v = t["V"][1][key].float().numpy()  # [nkv, d]
    if where == "window_outside":
        assert np.abs(row[0] - v[0]).max() > 0.5  # the strong key is just outside: it must not be seen
    else:
        np.testing.assert_allclose(row[0], v[0], atol=0.05)  # every head points at it
        np.testing.assert_allclose(row[3], v[1], atol=0.05)


def test_choose_splits():
    assert choose_splits(64, 8, 4096) == 4  # 512 CTAs would leave the second wave of 296 places 27 % empty; 2,048 fill seven
    assert choose_splits(64, 8, 4096, fill_last_wave=False) == 1
    assert choose_splits(8, 8, 4096) == 4
    assert choose_splits(1, 8, 4096) == 32
    assert choose_splits(1, 8, 100) == 1
    assert choose_splits(1000, 8, 100000) == 1


# ------------------------------------------------------------------ sampling


def test_greedy_takes_the_lowest_id_on_ties():
    logits = torch.zeros(3, 1000, device=DEV)
    logits[0, [17, 400, 999]] = 5.0
    logits[1, 999] = 1.0
    logits[2] = -float("inf")
    logits[2, 3] = -1e30
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.sample(out, logits)
    assert out.tolist() == [17, 999, 3]


def sample_rows(logits, temps, ks, ps, seeds, draws):
    n = logits.shape[0]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    mk = lambda v, dt: torch.tensor(v, dtype=dt, device=DEV)
    ops.sample(out, logits, mk(temps, torch.float32), mk(ks, torch.int32), mk(ps, torch.float32), mk(seeds, torch.int64), mk(draws, torch.int64))
    return out.tolist()


@pytest.mark.parametrize("V", [517, 5000, 10000, 20001, 128256])
def test_sampling_equals_the_plain_sampler(V):
    """Vocabularies that one CTA holds and ones that a cluster of 2, 4 and 8 shares (20,001: rows that do not
    start on a 16-byte boundary, and a last CTA with a shorter part)."""
    g = torch.Generator().manual_seed(V)
    logits = (torch.randn(24, V, generator=g) * 2.5).to(DEV)
    temps = [0.8, 1.0, 0.3, 2.0, 0.0, 1.3] * 4
    ks = [-1, 50, -1, 7, -1, 1] * 4
    ps = [1.0, 1.0, 0.9, 0.5, 1.0, 0.8] * 4
    seeds = [1234 + 77 * i for i in range(24)]
    draws = [i * 3 for i in range(24)]
    got = sample_rows(logits, temps, ks, ps, seeds, draws)
    host = logits.cpu().numpy()
    want = [plain.sample_token(host[i], temps[i], ks[i], ps[i], seeds[i], draws[i]) for i in range(24)]
    assert got == want


def test_a_rows_draw_does_not_depend_on_its_neighbours():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(8, 700, generator=g).to(DEV)
    alone = sample_rows(logits[2:3].contiguous(), [0.9], [-1], [0.95], [42], [5])
    busy = sample_rows(logits, [0.9] * 8, [-1] * 8, [0.95] * 8, [1, 2, 42, 4, 5, 6, 7, 8], [5] * 8)
    assert busy[2] == alone[0]


def test_sampled_frequencies_follow_the_distribution():
    probs = np.array([0.5, 0.25, 0.125, 0.125])
    logits = torch.tensor(np.log(probs), dtype=torch.float32, device=DEV).repeat(4000, 1)
    toks = sample_rows(logits, [1.0] * 4000, [-1] * 4000, [1.0] * 4000, [9] * 4000, list(range(4000)))
    freq = np.bincount(toks, minlength=4) / 4000
    assert np.abs(freq - probs).max() < 0.03
    # top_k = 2 renormalises over the two best; a tiny top_p leaves only the best
    toks = sample_rows(logits, [1.0] * 4000, [2] * 4000, [1.0] * 4000, [9] * 4000, list(range(4000)))
    freq = np.bincount(toks, minlength=4) / 4000
    assert freq[2:].sum() == 0 and abs(freq[0] - 2 / 3) < 0.03
    toks = sample_rows(logits[:50].contiguous(), [1.0] * 50, [-1] * 50, [0.01] * 50, [9] * 50, list(range(50)))
    assert set(toks) == {0}
    # ties at the k-th value are all kept: top_k = 2 of (0.4, 0.2, 0.2, 0.2) leaves the distribution as it is
    probs = np.array([0.4, 0.2, 0.2, 0.2])
    logits = torch.tensor(np.log(probs), dtype=torch.float32, device=DEV).repeat(4000, 1)
    toks = sample_rows(logits, [1.0] * 4000, [2] * 4000, [1.0] * 4000, [5] * 4000, list(range(4000)))
    assert np.abs(np.bincount(toks, minlength=4) / 4000 - probs).max() < 0.03


def test_a_vocabulary_too_large_for_temperature_sampling_is_refused_and_greedy_still_works():
    V = ops.SAMPLE_MAX_VOCAB_STOCHASTIC + 1
    logits = torch.zeros(2, V, device=DEV)
    logits[0, V - 1] = logits[1, 12345] = 3.0
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    ops.sample(out, logits)
    assert out.tolist() == [V - 1, 12345]
    with pytest.raises(ops.KernelError, match="temperature sampling takes vocabularies of up to"):
        sample_rows(logits, [1.0, 1.0], [-1, -1], [1.0, 1.0], [1, 2], [0, 0])
    edge = logits[:, : ops.SAMPLE_MAX_VOCAB_STOCHASTIC].contiguous()  # the largest one that is taken: 47 K floats a CTA
    edge[0, 77] = 40.0
    assert sample_rows(edge, [1.0, 0.0], [-1, -1], [1.0, 1.0], [1, 2], [0, 0]) == [77, 12345]


def test_sampling_in_a_large_vocabulary_finds_far_tokens_and_cuts_at_the_right_one():
    """128,256 logits shared by eight CTAs: the kept tokens lie in different CTAs' parts, so the cut, the totals and
    the draw all cross the cluster.  Five tokens hold nearly all the mass (0.4, 0.3, 0.15, 0.1, 0.05 of it)."""
    V, n = 128256, 3000
    ids = [128255, 7, 64000, 16032, 99999]
    probs = np.array([0.4, 0.3, 0.15, 0.1, 0.05])
    row = torch.full((V,), -30.0)
    row[ids] = torch.tensor(np.log(probs), dtype=torch.float32)
    logits = row.to(DEV).repeat(n, 1)
    def freq(k, p):
        toks = sample_rows(logits, [1.0] * n, [k] * n, [p] * n, [3] * n, list(range(n)))
        assert set(toks) <= set(ids)
        return np.array([toks.count(i) for i in ids]) / n
    assert np.abs(freq(-1, 1.0) - probs).max() < 0.035
    f = freq(3, 1.0)  # the three best, renormalised
    assert f[3:].sum() == 0 and np.abs(f[:3] - probs[:3] / probs[:3].sum()).max() < 0.035
    f = freq(-1, 0.75)  # 0.4 + 0.3 < 0.75 <= 0.4 + 0.3 + 0.15: the third is the last one kept
    assert f[3:].sum() == 0 and np.abs(f[:3] - probs[:3] / probs[:3].sum()).max() < 0.035
    f = freq(4, 0.5)  # top-k keeps four, top-p of their mass (0.95): 0.4 < 0.475 <= 0.7: two
    assert f[2:].sum() == 0 and np.abs(f[:2] - probs[:2] / probs[:2].sum()).max() < 0.035


def test_sampling_by_state_slot_reads_the_table_and_advances_the_draws():
    """The engine's way of sampling: the five parameter arrays are tables indexed by each row's state slot, and the
    kernel itself counts a stochastic row's draw.  Rows in an order that is not the slots', one greedy row, one
    row with top_k = 1; against the same rows sampled with explicit values, three steps in a row."""
    from dli_b200.sampling import Sampler, SamplingParams

    V, slots = 700, [5, 0, 3, 6, 2]
    g = torch.Generator().manual_seed(3)
    sampler = Sampler(DEV, max_requests=8)
    params = [SamplingParams(temperature=0.9, seed=11), SamplingParams(temperature=0.0), SamplingParams(temperature=1.4, top_k=20, seed=12),
              SamplingParams(temperature=0.7, top_k=1, seed=13), SamplingParams(temperature=1.1, top_p=0.8, seed=14)]
    start = [0, 0, 7, 3, 100]  # draws made so far (a request that comes back after a preemption starts where it was)
    for slot, p, d in zip(slots, params, start):
        sampler.bind(slot, p, p.seed or 0, d)
    stochastic = [not p.greedy for p in params]
    for step in range(3):
        logits = (torch.randn(len(slots), V, generator=g) * 2.0).to(DEV)
        got = sampler.sample_slots_async(logits, slots, all_greedy=False).result()
        want = sample_rows(logits, [0.0 if p.greedy else p.temperature for p in params], [p.top_k for p in params], [p.top_p for p in params],
                           [p.seed or 0 for p in params], [d + step for d in start])
        assert got == want, f"step {step}"
    draws = sampler.state.draws.tolist()
    assert [draws[s] for s in slots] == [d + 3 * st for d, st in zip(start, stochastic)]  # greedy rows draw nothing
    assert draws[1] == draws[4] == draws[7] == 0  # slots nobody was bound to
    # a slot given to another request takes that request's values, not its predecessor's
    sampler.bind(5, SamplingParams(temperature=0.0), 0, 0)
    logits = (torch.randn(1, V, generator=g) * 2.0).to(DEV)
    assert sampler.sample_slots_async(logits, [5], all_greedy=False).result() == [int(logits[0].argmax())]


# ------------------------------------------------------------------ decode matrix product


@pytest.mark.parametrize("tokens,features,K", [(1, 200, 96), (5, 130, 40), (17, 1000, 104), (64, 384, 520), (100, 256, 64), (256, 77, 1032), (8, 4100, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_skinny_gemm(tokens, features, K, out_dtype):
    """Sizes that are no multiples of the 128 x 64 tile, one K slice and several (a cluster),
    against a float64 product."""
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=tokens)
    w = rnd(features, K, dtype=torch.bfloat16, seed=features, scale=0.1)
    want = (x.double() @ w.double().T).cpu().numpy()
    scale = np.abs(want).max()
    for slices in (None, 1, 2, 5, 8, 13, 16):
        for _ in range(2):
            got = ops.skinny_gemm(x, w, out_dtype, slices)
            assert got.dtype == out_dtype and tuple(got.shape) == (tokens, features)
            err = np.abs(got.double().cpu().numpy() - want).max()
            assert err <= (1e-5 if out_dtype == torch.float32 else 8e-3) * max(1.0, scale), (slices, err)
    assert ops.skinny_gemm_error() == 0


def test_skinny_gemm_refuses_what_it_cannot_do():
    x = rnd(4, 36, dtype=torch.bfloat16)
    w = rnd(8, 36, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.skinny_gemm(x, w)
    with pytest.raises(ops.KernelError):
        ops.skinny_gemm(rnd(300, 64, dtype=torch.bfloat16), rnd(8, 64, dtype=torch.bfloat16))


@pytest.mark.parametrize("tokens,I,K,slices_hint", [(1, 64, 96, 1), (8, 192, 200, 2), (33, 1024, 2048, 3), (64, 128, 520, 8)])
def test_skinny_gemm_with_swiglu_epilogue(tokens, I, K, slices_hint):
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=I)
    gate = rnd(I, K, dtype=torch.bfloat16, seed=I + 1, scale=0.1)
    up = rnd(I, K, dtype=torch.bfloat16, seed=I + 2, scale=0.1)
    tiled = torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], 1).reshape(2 * I, K).contiguous()
    got = ops.skinny_gemm_swiglu(x, tiled)
    g = x.double() @ gate.double().T
    u = x.double() @ up.double().T
    want = (plain.silu(g.cpu().numpy()) * u.cpu().numpy())
    np.testing.assert_allclose(got.double().cpu().numpy(), want, atol=8e-3 * max(1.0, np.abs(want).max()))
    # and the stand-alone kernel reads the same tiled layout
    gu = (x.float() @ tiled.float().T).to(torch.bfloat16)
    out = torch.empty(tokens, I, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(out, gu, tiled=True)
    np.testing.assert_allclose(out.double().cpu().numpy(), want, atol=2e-2 * max(1.0, np.abs(want).max()))
    assert ops.skinny_gemm_error() == 0


@pytest.mark.parametrize("nh,nkv,d,rot,page", [(5, 1, 64, 64, 8), (4, 2, 16, 16, 4), (3, 3, 32, 16, 16), (2, 1, 128, 128, 16), (6, 2, 64, 0, 32)])
def test_skinny_gemm_with_rotary_epilogue(nh, nkv, d, rot, page):
    """The fused projection + rotary + cache write against the separate kernels."""
    tokens, K, pages = 7, 264, 6
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=nh)
    w = rnd((nh + 2 * nkv) * d, K, dtype=torch.bfloat16, seed=d, scale=0.1)
    positions = torch.tensor([0, 1, 63, 64, 4095, 100000, 17], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 8, pages * page - 1, 0, 16, -1, 22], dtype=torch.int32, device=DEV)
    inv = torch.from_numpy(plain.inverse_frequencies({"head_dim": rot, "theta": 10000.0, "rope_type": "default"})).to(DEV) if rot else None
    kp1, vp1 = (torch.full((pages, nkv, page, d), 9.0, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    kp2, vp2 = kp1.clone(), vp1.clone()
    q = ops.skinny_gemm_rotary(x, w, positions, inv, slots, kp1, vp1, nh, nkv, d, rot, page, True)
    qkv = (x.float() @ w.float().T)  # float32 product, then the stand-alone kernel on its bfloat16 rounding
    ref = qkv.to(torch.bfloat16).contiguous()
    ops.rotary_store(ref, positions, inv, slots, kp2, vp2, nh, nkv, d, rot, page, True)
    t2 = 2e-2 * max(1.0, float(qkv.abs().max()))
    np.testing.assert_allclose(q.float().cpu().numpy(), ref[:, : nh * d].float().cpu().numpy(), atol=t2)
    np.testing.assert_allclose(kp1.float().cpu().numpy(), kp2.float().cpu().numpy(), atol=t2)
    np.testing.assert_allclose(vp1.float().cpu().numpy(), vp2.float().cpu().numpy(), atol=t2)
    assert ops.skinny_gemm_error() == 0


@pytest.mark.parametrize("tokens,H,K,slices", [(1, 128, 64, 1), (8, 2048, 2048, 8), (5, 200, 520, 3), (8, 264, 96, None), (33, 384, 1032, 2)])
def test_skinny_gemm_with_residual_epilogue_and_row_scaling(tokens, H, K, slices):
    """h += x W^T with the first half of the RMS norm in the epilogue, then the products that read
    the result (plain, SiLU * up, float32 logits) and apply the norm's row factor, against the
    formulas in float64.  One row of h is tiny and eps large, so a dropped eps would show."""
    eps = 1e-3
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=tokens)
    w = rnd(H, K, dtype=torch.bfloat16, seed=H, scale=0.05)
    h0 = rnd(tokens, H, seed=K)
    h0[0] *= 1e-3
    x[0] *= 1e-3
    gain = (1.0 + 0.3 * rnd(H, seed=3)).contiguous()
    h = h0.clone()
    got = ops.skinny_gemm_residual(x, w, h, gain, eps, slices)
    want_h = h0.double() + x.double() @ w.double().T
    np.testing.assert_allclose(h.double().cpu().numpy(), want_h.cpu().numpy(), atol=1e-4 * max(1.0, float(want_h.abs().max())))
    assert tuple(got.ssq.shape) == (tokens, (H + 127) // 128)
    np.testing.assert_allclose(got.ssq.double().sum(1).cpu().numpy(), (want_h ** 2).sum(1).cpu().numpy(), rtol=1e-4)
    np.testing.assert_allclose(got.x.double().cpu().numpy(), (want_h * gain.double()).cpu().numpy(),
                               atol=8e-3 * max(1.0, float((want_h * gain.double()).abs().max())))
    # the readers: y = rmsnorm(h) * gain, then products of y
    rstd = 1.0 / torch.sqrt((want_h ** 2).mean(1, keepdim=True) + eps)
    y = want_h * rstd * gain.double()
    w2 = rnd(136, H, dtype=torch.bfloat16, seed=7, scale=0.1)
    for out_dtype, tol in ((torch.bfloat16, 2e-2), (torch.float32, 1e-2)):
        for sl in (None, 1, 4):
            out = ops.skinny_gemm(got, w2, out_dtype, sl)
            want = (y @ w2.double().T).cpu().numpy()
            np.testing.assert_allclose(out.double().cpu().numpy(), want, atol=tol * max(1.0, np.abs(want).max()))
    I = 128
    gate = rnd(I, H, dtype=torch.bfloat16, seed=8, scale=0.1)
    up = rnd(I, H, dtype=torch.bfloat16, seed=9, scale=0.1)
    tiled = torch.stack([gate.view(I // 64, 64, H), up.view(I // 64, 64, H)], 1).reshape(2 * I, H).contiguous()
    act = ops.skinny_gemm_swiglu(got, tiled)
    want = plain.silu((y @ gate.double().T).cpu().numpy()) * (y @ up.double().T).cpu().numpy()
    np.testing.assert_allclose(act.double().cpu().numpy(), want, atol=2e-2 * max(1.0, np.abs(want).max()))
    # a second residual product reading the first one's rows
    w3 = rnd(H, H, dtype=torch.bfloat16, seed=11, scale=0.05)
    h2 = h.clone()
    nxt = ops.skinny_gemm_residual(got, w3, h2, gain, eps)
    want_h2 = h.double() + y @ w3.double().T
    np.testing.assert_allclose(h2.double().cpu().numpy(), want_h2.cpu().numpy(), atol=2e-2 * max(1.0, float(want_h2.abs().max())))
    np.testing.assert_allclose(nxt.ssq.double().sum(1).cpu().numpy(), (h2.double() ** 2).sum(1).cpu().numpy(), rtol=1e-4)
    assert ops.skinny_gemm_error() == 0


# ------------------------------------------------------------------ matrix product of many tokens


@pytest.mark.parametrize("tokens,features,K", [(1, 8, 8), (128, 256, 64), (130, 264, 72), (517, 1000, 136), (2048, 3072, 2048), (300, 20000, 520), (5000, 384, 264)])
def test_dense_gemm(tokens, features, K):
    """Sizes on and off the 128 x 256 x 64 tile, fewer tiles than SMs and many per CTA (both accumulators in turn,
    every stage reused), against a float64 product."""
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=tokens)
    w = rnd(features, K, dtype=torch.bfloat16, seed=features, scale=0.1)
    want = (x.double() @ w.double().T).cpu().numpy()
    for _ in range(2):
        got = ops.dense_gemm(x, w)
        assert got.dtype == torch.bfloat16 and tuple(got.shape) == (tokens, features)
        err = np.abs(got.double().cpu().numpy() - want).max()
        assert err <= 8e-3 * max(1.0, np.abs(want).max()), err
    assert ops.dense_gemm_error() == 0


def test_dense_gemm_refuses_what_it_cannot_do():
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.dense_gemm(rnd(4, 36, dtype=torch.bfloat16), rnd(8, 36, dtype=torch.bfloat16))
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.dense_gemm(rnd(4, 64, dtype=torch.bfloat16), rnd(12, 64, dtype=torch.bfloat16))
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.dense_gemm_rotary(rnd(4, 64, dtype=torch.bfloat16), rnd(4 * 80, 64, dtype=torch.bfloat16), None, None, None, None, 2, 1, 80, 0, 16, False)


@pytest.mark.parametrize("tokens,I,K", [(1, 64, 96), (129, 192, 200), (700, 1024, 2048), (2048, 8192, 264)])
def test_dense_gemm_with_swiglu_epilogue(tokens, I, K):
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=I)
    gate = rnd(I, K, dtype=torch.bfloat16, seed=I + 1, scale=0.1)
    up = rnd(I, K, dtype=torch.bfloat16, seed=I + 2, scale=0.1)
    tiled = torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], 1).reshape(2 * I, K).contiguous()
    got = ops.dense_gemm_swiglu(x, tiled)
    assert tuple(got.shape) == (tokens, I)
    g = (x.double() @ gate.double().T).cpu().numpy()
    u = (x.double() @ up.double().T).cpu().numpy()
    want = plain.silu(g) * u
    np.testing.assert_allclose(got.double().cpu().numpy(), want, atol=8e-3 * max(1.0, np.abs(want).max()))
    assert ops.dense_gemm_error() == 0


@pytest.mark.parametrize("nh,nkv,d,rot,page,tokens", [(5, 1, 64, 64, 8, 7), (2, 1, 128, 128, 16, 300), (3, 2, 128, 64, 16, 131), (6, 2, 64, 0, 32, 257), (32, 8, 64, 64, 16, 600)])
def test_dense_gemm_with_rotary_epilogue(nh, nkv, d, rot, page, tokens):
    """The fused projection + rotary + cache write against the separate kernels: heads of 64 and 128, whole, partial
    and no rotation, tokens without a slot, more heads than a tile holds."""
    K = 264
    pages = tokens // page + 3
    x = rnd(tokens, K, dtype=torch.bfloat16, seed=nh)
    w = rnd((nh + 2 * nkv) * d, K, dtype=torch.bfloat16, seed=d, scale=0.1)
    g = torch.Generator().manual_seed(tokens)
    positions = torch.randint(0, 100000, (tokens,), generator=g).to(torch.int32).to(DEV)
    slots = torch.randperm(pages * page, generator=g)[:tokens].to(torch.int32)
    slots[3 % tokens] = -1
    slots = slots.to(DEV)
    inv = torch.from_numpy(plain.inverse_frequencies({"head_dim": rot, "theta": 10000.0, "rope_type": "default"})).to(DEV) if rot else None
    table = ops.rotary_table(positions, inv) if rot else None
    kp1, vp1 = (torch.full((pages, nkv, page, d), 9.0, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    kp2, vp2 = kp1.clone(), vp1.clone()
    q = ops.dense_gemm_rotary(x, w, table, slots, kp1, vp1, nh, nkv, d, rot, page, True)
    qkv = (x.float() @ w.float().T)  # float32 product, then the stand-alone kernel on its bfloat16 rounding
    ref = qkv.to(torch.bfloat16).contiguous()
    ops.rotary_store(ref, positions, inv, slots, kp2, vp2, nh, nkv, d, rot, page, True)
    t2 = 2e-2 * max(1.0, float(qkv.abs().max()))
    np.testing.assert_allclose(q.float().cpu().numpy(), ref[:, : nh * d].float().cpu().numpy(), atol=t2)
    np.testing.assert_allclose(kp1.float().cpu().numpy(), kp2.float().cpu().numpy(), atol=t2)
    np.testing.assert_allclose(vp1.float().cpu().numpy(), vp2.float().cpu().numpy(), atol=t2)
    # without the cache write the pools stay as they are
    kp3, vp3 = kp1.clone(), vp1.clone()
    q2 = ops.dense_gemm_rotary(x, w, table, None, None, None, nh, nkv, d, rot, page, False)
    assert torch.equal(q, q2) and torch.equal(kp3, kp1) and torch.equal(vp3, vp1)
    assert ops.dense_gemm_error() == 0


def test_a_wait_inside_the_many_token_product_runs_out_and_both_ctas_give_up_in_order():
    """Neither CTA of the pair issues the copies of the last k step (a test-only entry; a flag that nothing sets) and
    the waits are limited to a few thousand polls: the waits for those operands and for the accumulator run out, the
    first one's code is recorded, both CTAs reach the end together and free their tensor memory.  The host reads the
    code, nothing hangs, and the next ordinary product of the same shapes is right."""
    tokens, features, K = 200, 256, 320  # one tile, five k steps, each in a stage of its own
    x, w = rnd(tokens, K, dtype=torch.bfloat16, seed=1), rnd(features, K, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = (x.float() @ w.float().T).cpu().numpy()
    assert ops.device_wait_errors() == {}
    ops.dense_gemm_wait_test(x, w, wait_limit=4000)
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    assert ops.dense_gemm_error() in (3, 4)
    found = ops.device_wait_errors()
    assert found.get("dense_gemm.cu") in (3, 4) and ops.device_wait_errors() == {}  # read once, then forgotten
    for _ in range(3):
        got = ops.dense_gemm(x, w)
        np.testing.assert_allclose(got.float().cpu().numpy(), want, atol=2e-2)
    assert ops.dense_gemm_error() == 0


def test_a_wait_inside_the_decode_product_runs_out_and_the_kernel_gives_up_in_order():
    """The copies of one k tile are never issued (a test-only entry; a flag that nothing sets) and the waits are
    limited to a few thousand polls: the kernel gives the wait up, records which one it was, completes its cluster
    barriers, frees its tensor memory and returns.  The host reads the code, nothing hangs, and the next
    ordinary product — same shapes, same cluster size, tensor memory allocated afresh — is right."""
    tokens, features, K, slices = 5, 384, 512, 2  # 8 k tiles: 4 per slice, each in a stage of its own
    x, w = rnd(tokens, K, dtype=torch.bfloat16, seed=1), rnd(features, K, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.float() @ w.float().T
    assert ops.device_wait_errors() == {}
    ops.skinny_gemm_wait_test(x, w, slices, wait_limit=4000, skip_tile=7)  # the last tile of the second slice never arrives
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    assert ops.skinny_gemm_error() == 2  # the tensor-core warp's wait for a stage's copies
    assert ops.device_wait_errors() == {"skinny_gemm.cu": 2} and ops.device_wait_errors() == {}  # read once, then forgotten
    for _ in range(3):
        got = ops.skinny_gemm(x, w, out_dtype=torch.float32, slices=slices)
        np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), atol=2e-2)
    assert ops.skinny_gemm_error() == 0
