"""Rotary position encoding (rotate-half pairing) with default, linear and llama3 frequency scaling."""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..kernels.gemm import dense_product, fused_epilogue, project
from .base import Part, register_part


def inverse_frequencies(params) -> torch.Tensor:
    """[rotary_dim / 2] float32 on the CPU, every step in float32 as the reference does it
    (src/dli/model/rope.py:21-47): exponents 2j/d, 1 / theta**e; ``linear`` divides every
    frequency by ``factor`` (positions are interpolated); for ``llama3`` wavelengths
    beyond original_max / low_freq_factor are divided by ``factor``, those under
    original_max / high_freq_factor kept, and the band between interpolated."""
    d = int(params["rotary_dim"])
    exponents = torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d
    inv = 1.0 / (float(params["theta"]) ** exponents)
    scaling = params.get("scaling", "default")
    if scaling == "default":
        return inv
    if scaling == "linear":
        return inv / float(params["factor"])
    if scaling != "llama3":
        raise ValueError(f"rotary scaling {scaling!r} is not supported (default, linear, llama3)")
    old = params["original_max_position_embeddings"]
    factor, low, high = float(params["factor"]), float(params["low_freq_factor"]), float(params["high_freq_factor"])
    wavelen = 2 * math.pi / inv
    scaled = torch.where(wavelen > old / low, inv / factor, inv)
    smooth = (old / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < old / high) & ~(wavelen > old / low)
    return torch.where(medium, smoothed, scaled)


def _step_table(batch, inv_freq, table_key):
    """The sines and cosines of the step's tokens, computed once and shared by all layers with these frequencies."""
    key = ("rotary_table", table_key)
    table = batch.scratch.get(key)
    if table is None:
        table = batch.scratch[key] = ops.rotary_table(batch.positions, inv_freq)
    return table


def _rotate_and_store(qkv, batch, cache, num_heads, num_kv_heads, write_kv, head_dim, rotary_dim, inv_freq, table_key=None):
    """Runs the fused kernel and returns the tensor whose leading num_heads * head_dim columns
    are the encoded queries (qkv itself: queries are rotated in place)."""
    group = batch.group(cache.group)
    args = (batch.positions, inv_freq, group.slots if write_kv else None, cache.k if write_kv else None,
            cache.v if write_kv else None, num_heads, num_kv_heads, head_dim, rotary_dim, cache.page_size, write_kv)
    if rotary_dim or write_kv:
        many = rotary_dim and qkv.dtype == torch.bfloat16 and qkv.shape[0] > 64
        ops.rotary_store(qkv, *args, table=_step_table(batch, inv_freq, table_key) if many else None)
    return qkv


def _project_and_encode(x, wqkv, batch, cache, num_heads, num_kv_heads, write_kv, head_dim, rotary_dim, inv_freq, table_key=None):
    """q | k | v projection followed by position encoding and cache write; for a decode step's few
    tokens and for a long portion's many both happen in one kernel (the product's epilogue rotates and
    writes the cache)."""
    if fused_epilogue(x) and ops.skinny_rotary_supported(head_dim):
        group = batch.group(cache.group)
        return ops.skinny_gemm_rotary(x, wqkv, batch.positions, inv_freq, group.slots, cache.k, cache.v, num_heads, num_kv_heads,
                                      head_dim, rotary_dim, cache.page_size, write_kv)
    if ops.dense_rotary_supported(head_dim, rotary_dim) and dense_product(x, wqkv.shape[0], "rotary"):
        group = batch.group(cache.group)
        table = _step_table(batch, inv_freq, table_key) if rotary_dim else None
        return ops.dense_gemm_rotary(x, wqkv, table, group.slots if write_kv else None, cache.k if write_kv else None,
                                     cache.v if write_kv else None, num_heads, num_kv_heads, head_dim, rotary_dim, cache.page_size, write_kv)
    return _rotate_and_store(project(x, wqkv), batch, cache, num_heads, num_kv_heads, write_kv, head_dim, rotary_dim, inv_freq, table_key)


@register_part("position", "rotary")
class Rotary(Part):
    """params: head_dim, rotary_dim (<= head_dim; elements beyond it pass through), theta,
    scaling and its constants.  The angle float32(position) * inv_freq and its sine and cosine
    are computed in float32 inside the kernel that also writes k and v to the cache."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and at most head_dim={self.head_dim}")
        inv = inverse_frequencies(spec.params) if self.rotary_dim else None
        self.inv_freq = inv.to(env.device) if inv is not None else None
        # layers with the same frequencies share one table of sines and cosines per step
        self.table_key = hash(tuple(inv.tolist())) if inv is not None else None

    def rotate_and_store(self, qkv, batch, cache, num_heads: int, num_kv_heads: int, write_kv: bool):
        return _rotate_and_store(qkv, batch, cache, num_heads, num_kv_heads, write_kv, self.head_dim, self.rotary_dim, self.inv_freq, self.table_key)

    def project_and_encode(self, x, wqkv, batch, cache, num_heads: int, num_kv_heads: int, write_kv: bool):
        return _project_and_encode(x, wqkv, batch, cache, num_heads, num_kv_heads, write_kv, self.head_dim, self.rotary_dim, self.inv_freq, self.table_key)


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q passes through, k and v are written to the cache as they are."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])

    def rotate_and_store(self, qkv, batch, cache, num_heads: int, num_kv_heads: int, write_kv: bool):
        return _rotate_and_store(qkv, batch, cache, num_heads, num_kv_heads, write_kv, self.head_dim, 0, None)

    def project_and_encode(self, x, wqkv, batch, cache, num_heads: int, num_kv_heads: int, write_kv: bool):
        return _project_and_encode(x, wqkv, batch, cache, num_heads, num_kv_heads, write_kv, self.head_dim, 0, None)
