"""Stand-ins for the kernels, written with torch on the CPU, for tests of the engine's host side.

The product has no CPU path.  These functions exist only so that the Python above the kernels
(parts and their wiring, batch building, cache pools, the step function, scheduler, engine, the
step launched ahead) can run end to end in the CPU test suite and be compared with the plain
implementation.  Each one restates what its kernel's wrapper documents (kernels/ops.py); none is
used by the GPU tests, which run the real kernels.  ``patched()`` swaps them in.
"""

from __future__ import annotations

import contextlib

import numpy as np
import torch

from dli_b200.engine import graphs as graphs_mod
from dli_b200.engine import runner as runner_mod
from dli_b200.kernels import gemm, ops
from dli_b200.parts import model as model_mod
from tests.plain import llama_plain as plain


def embedding(h, table, ids):
    h.copy_(table[ids.long()].float())


def patch_tokens(ids, source, src):
    pick = src >= 0
    ids[pick] = source[src[pick].long()]


def copy_page(pool, src, dst):
    pool[:, dst] = pool[:, src]


def add_rmsnorm(y, h, delta, weight, eps, rows=None):
    if rows is None:
        if delta is not None:
            h += delta.float()
        x = h
    else:
        x = h[rows.long()] + (delta[rows.long()].float() if delta is not None else 0.0)
    y.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight).to(y.dtype))


def rotary_table(positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], -1)


def rotary_store(qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim, page_size,
                 write_kv=True, table=None):
    n = qkv.shape[0]
    heads = qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)
    if rotary_dim:
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        qk = heads[:, : num_heads + num_kv_heads, :rotary_dim].float()
        lo, hi = qk[..., :half].clone(), qk[..., half:].clone()
        heads[:, : num_heads + num_kv_heads, :half] = (lo * cos - hi * sin).to(qkv.dtype)
        heads[:, : num_heads + num_kv_heads, half:rotary_dim] = (hi * cos + lo * sin).to(qkv.dtype)
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = heads[:, num_heads : num_heads + num_kv_heads]
        v_pool[page, :, off, :] = heads[:, num_heads + num_kv_heads :]


def silu_mul(out, gate_up, tiled=False):
    n, inter = out.shape
    if tiled:
        blocks = gate_up.view(n, inter // 64, 2, 64)
        gate, up = blocks[:, :, 0].reshape(n, inter), blocks[:, :, 1].reshape(n, inter)
    else:
        gate, up = gate_up[:, :inter], gate_up[:, inter:]
    g = gate.float()
    out.copy_((g / (1 + torch.exp(-g)) * up.float()).to(out.dtype))


def paged_attention_simt(out, qkv, k_pool, v_pool, block_tables, seq_of_token, positions, num_heads, scale, window=None):
    n = out.shape[0]
    _, nkv, page_size, d = k_pool.shape
    fan = num_heads // nkv
    q = qkv[:, : num_heads * d].view(n, num_heads, d).float()
    for t in range(n):
        p = int(positions[t])
        first = max(0, p - window + 1) if window else 0
        keys = torch.arange(first, p + 1)
        table = block_tables[int(seq_of_token[t])]
        pages = table[(keys // page_size).long()].long()
        assert (pages >= 0).all(), "attention reads a page that was given back"
        k = k_pool[pages, :, (keys % page_size).long(), :].float()  # [keys, nkv, d]
        v = v_pool[pages, :, (keys % page_size).long(), :].float()
        k, v = k.repeat_interleave(fan, 1), v.repeat_interleave(fan, 1)  # [keys, nh, d]
        s = torch.einsum("hd,khd->hk", q[t], k) * scale
        w = torch.softmax(s, -1)
        out[t] = torch.einsum("hk,khd->hd", w, v).reshape(-1).to(out.dtype)


def _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window):
    """The bfloat16 attention kernels' common contract: sequences [seq0, seq0 + num_seqs); a sequence's
    tokens sit in rows q_start[s] .. q_start[s + 1] at positions kv_len[s] - q_len .. kv_len[s] - 1."""
    rows, seqs, pos = [], [], []
    for s in range(seq0, seq0 + num_seqs):
        lo, hi = int(q_start[s]), int(q_start[s + 1])
        rows += range(lo, hi)
        seqs += [s] * (hi - lo)
        pos += range(int(kv_len[s]) - (hi - lo), int(kv_len[s]))
    if not rows:
        return
    idx = torch.tensor(rows)
    part = torch.empty((len(rows), out.shape[1]), dtype=out.dtype)
    paged_attention_simt(part, qkv[idx], k_pool, v_pool, block_tables, torch.tensor(seqs, dtype=torch.int32),
                         torch.tensor(pos, dtype=torch.int32), num_heads, scale, window)
    out[idx] = part


def paged_attention_mma(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, max_q_len, first_row, num_heads, scale,
                        window=None, splits=1, scratch=None):
    assert splits == 1 or (max_q_len == 1 and scratch is not None)
    _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window)


def paged_decode_tma(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, first_row, num_heads, scale,
                     window=None, splits=1, scratch=None, max_kv_len=0):
    assert splits == 1 or scratch is not None
    _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window)


def paged_prefill_tc(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, max_q_len, num_heads, scale,
                     window=None, query_tiles=0):
    _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window)


# ---- the decode matrix product and its epilogues (bfloat16 in, float32 sums)


def _sums(x, weight):
    """float32 sums of x W^T; x may be ops.ScaledRows, whose row factor is applied to the sums."""
    if isinstance(x, ops.ScaledRows):
        factor = torch.rsqrt(x.ssq.sum(-1, keepdim=True) / x.x.shape[1] + x.eps)
        return (x.x.float() @ weight.float().t()) * factor
    return x.float() @ weight.float().t()


def skinny_gemm_slices(tokens, features, in_features):
    return 1


def skinny_gemm(x, weight, out_dtype=torch.bfloat16, slices=None, out=None, max_stages=0):
    y = _sums(x, weight).to(out_dtype)
    if out is None:
        return y
    out.copy_(y)
    return out


def skinny_gemm_residual(x, weight, h, gain, eps, slices=None):
    h += _sums(x, weight)
    tokens, features = h.shape
    tiles = -(-features // 128)
    sq = torch.zeros((tokens, tiles * 128))
    sq[:, :features] = h * h
    return ops.ScaledRows((h * gain).to(torch.bfloat16), sq.view(tokens, tiles, 128).sum(-1), eps)


def skinny_gemm_swiglu(x, weight_tiled):
    y = _sums(x, weight_tiled)
    out = torch.empty((y.shape[0], y.shape[1] // 2), dtype=torch.bfloat16)
    silu_mul(out, y, tiled=True)
    return out


def skinny_gemm_rotary(x, wqkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim, page_size, write_kv):
    qkv = _sums(x, wqkv)  # rotated in float32, rounded once (as the kernel's epilogue does)
    pools = (torch.empty_like(k_pool, dtype=torch.float32), torch.empty_like(v_pool, dtype=torch.float32)) if write_kv else (None, None)
    rotary_store(qkv, positions, inv_freq, slots, pools[0], pools[1], num_heads, num_kv_heads, head_dim, rotary_dim, page_size, write_kv)
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = pools[0][page, :, off, :].to(k_pool.dtype)
        v_pool[page, :, off, :] = pools[1][page, :, off, :].to(v_pool.dtype)
    return qkv[:, : num_heads * head_dim].to(torch.bfloat16)


# ---- the product of many tokens and its epilogues


def dense_gemm(x, weight, out=None):
    return skinny_gemm(x, weight, torch.bfloat16, out=out)


def dense_gemm_swiglu(x, weight_tiled):
    return skinny_gemm_swiglu(x, weight_tiled)


def dense_gemm_rotary(x, wqkv, table, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim, page_size, write_kv):
    qkv = _sums(x, wqkv)
    n = qkv.shape[0]
    heads = qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)
    if rotary_dim:
        half = rotary_dim // 2
        cos, sin = table[:, None, :half], table[:, None, half:]
        qk = heads[:, : num_heads + num_kv_heads, :rotary_dim]
        lo, hi = qk[..., :half].clone(), qk[..., half:].clone()
        heads[:, : num_heads + num_kv_heads, :half] = lo * cos - hi * sin
        heads[:, : num_heads + num_kv_heads, half:rotary_dim] = hi * cos + lo * sin
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = heads[:, num_heads : num_heads + num_kv_heads].to(k_pool.dtype)
        v_pool[page, :, off, :] = heads[:, num_heads + num_kv_heads :].to(v_pool.dtype)
    return qkv[:, : num_heads * head_dim].to(torch.bfloat16)


def sample(out, logits, temperature=None, top_k=None, top_p=None, seed=None, draw=None):
    rows = logits.shape[0]
    for r in range(rows):
        row = logits[r].numpy()
        if temperature is None:
            out[r] = int(np.argmax(row))
        else:
            out[r] = plain.sample_token(row, float(temperature[r]), int(top_k[r]), float(top_p[r]), int(seed[r]), int(draw[r]))


def linear(x, weight, out=None):
    return torch.matmul(x, weight.t(), out=out)


class CpuPending:
    def __init__(self, ids: torch.Tensor) -> None:
        self.device_ids = ids
        self.reads = 0

    def result(self) -> list[int]:
        self.reads += 1
        return self.device_ids.tolist()


class CpuSampler:
    """The engine's Sampler without pinned memory and events: same calls, same keys (seed, draw)."""

    def _run(self, logits, params, seeds, draws) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32)
        if all(p.greedy for p in params):
            sample(out, logits)
        else:
            sample(out, logits, [0.0 if p.greedy else p.temperature for p in params], [p.top_k for p in params],
                   [p.top_p for p in params], list(seeds), list(draws))
        return out

    def sample(self, logits, params, seeds, draws) -> list[int]:
        return self._run(logits, params, seeds, draws).tolist() if logits.shape[0] else []

    def sample_async(self, logits, params, seeds, draws) -> CpuPending:
        return CpuPending(self._run(logits, params, seeds, draws))


OPS = {"embedding": embedding, "patch_tokens": patch_tokens, "copy_page": copy_page, "add_rmsnorm": add_rmsnorm,
       "rotary_table": rotary_table, "rotary_store": rotary_store, "silu_mul": silu_mul, "paged_attention_simt": paged_attention_simt,
       "paged_attention_mma": paged_attention_mma, "paged_decode_tma": paged_decode_tma, "paged_prefill_tc": paged_prefill_tc,
       "skinny_gemm_slices": skinny_gemm_slices, "skinny_gemm": skinny_gemm, "skinny_gemm_residual": skinny_gemm_residual,
       "skinny_gemm_swiglu": skinny_gemm_swiglu, "skinny_gemm_rotary": skinny_gemm_rotary, "dense_gemm": dense_gemm,
       "dense_gemm_swiglu": dense_gemm_swiglu, "dense_gemm_rotary": dense_gemm_rotary,
       "sample": sample}


calls: dict[str, int] = {}  # how often each stand-in ran since patched() was entered


def _counted(name, fn):
    def run(*args, **kwargs):
        calls[name] = calls.get(name, 0) + 1
        return fn(*args, **kwargs)

    return run


@contextlib.contextmanager
def patched():
    """Inside: models on ``device='cpu'`` build, load and step through the stand-ins (float32, and bfloat16
    with the decode products' fused epilogues)."""
    saved = {name: getattr(ops, name) for name in OPS}
    saved_linear, saved_model_linear, saved_require = gemm.linear, model_mod.linear, runner_mod._require_cuda
    saved_lookup, saved_mixed = graphs_mod.DecodeGraphs.lookup, graphs_mod.DecodeGraphs.lookup_mixed
    try:
        graphs_mod.DecodeGraphs.lookup = graphs_mod.DecodeGraphs.lookup_mixed = lambda self, *a, **k: None  # no captured steps without a device
        calls.clear()
        for name, fn in OPS.items():
            setattr(ops, name, _counted(name, fn))
        gemm.linear = model_mod.linear = linear
        runner_mod._require_cuda = lambda device: None
        yield
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
        gemm.linear, model_mod.linear, runner_mod._require_cuda = saved_linear, saved_model_linear, saved_require
        graphs_mod.DecodeGraphs.lookup, graphs_mod.DecodeGraphs.lookup_mixed = saved_lookup, saved_mixed

