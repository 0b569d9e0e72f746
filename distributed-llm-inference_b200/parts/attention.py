"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import torch

from ..cache.needs import PagedKVNeed
from ..kernels import attention as attn_kernels
from ..kernels.gemm import last_product, project
from ..weights.loader import TensorDecl
from .base import Part, build_part, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q, k, v projections, position encoding, causal attention of each token over the keys of
    its own sequence at positions <= its own (optionally only the last ``window``), output
    projection (src/dli/model/llama.py:72-76,94-95,147-177).  Query head h reads kv head
    h // (num_heads / num_kv_heads).  The three projection matrices are read by their own
    names and laid side by side at load, so one product yields q | k | v.

    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window, position (PartSpec).
    """

    graph_capturable = True
    takes_scaled_rows = True  # the input only goes to the q | k | v product
    defer_output = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        if self.nh % self.nkv:
            raise ValueError(f"num_heads={self.nh} is not a multiple of num_kv_heads={self.nkv}")
        self.position = build_part("position", p["position"], env)
        self.wqkv: torch.Tensor | None = None
        self.wo: torch.Tensor | None = None

    def children(self):
        return [self.position]

    def declare(self):
        px, H, d = self.spec.prefix, self.hidden, self.d
        return {
            px + "q_proj.weight": TensorDecl((self.nh * d, H)),
            px + "k_proj.weight": TensorDecl((self.nkv * d, H)),
            px + "v_proj.weight": TensorDecl((self.nkv * d, H)),
            px + "o_proj.weight": TensorDecl((H, self.nh * d)),
        }

    def load(self, tensors):
        px = self.spec.prefix
        self.wqkv = torch.cat([tensors[px + "q_proj.weight"], tensors[px + "k_proj.weight"], tensors[px + "v_proj.weight"]], 0).contiguous()
        self.wo = tensors[px + "o_proj.weight"]

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        """Into how many runs the decode kernel cuts each sequence's keys (1: not at all)."""
        return attn_kernels.decode_splits(num_seqs, self.nh, self.nkv, self.d, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        encode = getattr(self.position, "project_and_encode", None)
        if encode is not None:  # the position part may fuse the projection with its encoding
            q = encode(x, self.wqkv, batch, cache, self.nh, self.nkv, cache.writes)
        else:
            q = self.position.rotate_and_store(project(x, self.wqkv), batch, cache, self.nh, self.nkv, cache.writes)
        out = torch.empty((x.shape[0], self.nh * self.d), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(out, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)))
        return last_product(out, self.wo, self.defer_output)
