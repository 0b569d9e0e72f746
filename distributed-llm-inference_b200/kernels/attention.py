"""Chooses the attention kernels of a step.

float32: the CUDA-core kernel for every token (true 32-bit).  bfloat16: tensor-core
kernels where the head size has one — the split-key decode kernel for sequences that
bring one token, the tiled prefill kernel for longer portions — and the CUDA-core
kernel otherwise (windowed attention, head sizes that are no multiple of 16).
"""

from __future__ import annotations

import torch

from . import ops


def paged_attention(out: torch.Tensor, qkv: torch.Tensor, cache, batch, num_heads: int, scale: float, window: int | None) -> None:
    group = batch.group(cache.group)
    ops.paged_attention_simt(out, qkv, cache.k, cache.v, group.block_tables, batch.seq_of_token, batch.positions,
                             num_heads, scale, window)
