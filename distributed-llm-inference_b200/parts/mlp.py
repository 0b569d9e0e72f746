"""SwiGLU feed-forward."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.gemm import dense_product, fused_epilogue, last_product, project
from ..weights.loader import TensorDecl
from .base import Part, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)) (src/dli/model/llama.py:189-191).  gate and up are read by
    their own names and laid together at load, so one product yields both: side by side, or —
    when the intermediate size is a multiple of 64 — interleaved in blocks of 64 rows, the layout
    in which the decode product applies SiLU(gate) * up in its own epilogue.
    params: hidden_size, intermediate_size."""

    graph_capturable = True
    takes_scaled_rows = True  # the input only goes to the gate | up product
    defer_output = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up: torch.Tensor | None = None
        self.tiled = False
        self.w_down: torch.Tensor | None = None

    def declare(self):
        px = self.spec.prefix
        return {
            px + "gate_proj.weight": TensorDecl((self.inter, self.hidden)),
            px + "up_proj.weight": TensorDecl((self.inter, self.hidden)),
            px + "down_proj.weight": TensorDecl((self.hidden, self.inter)),
        }

    def load(self, tensors):
        px = self.spec.prefix
        gate, up = tensors[px + "gate_proj.weight"], tensors[px + "up_proj.weight"]
        self.tiled = self.inter % 64 == 0 and self.env.dtype == torch.bfloat16
        if self.tiled:
            blocks = self.inter // 64
            self.w_gate_up = torch.stack([gate.view(blocks, 64, self.hidden), up.view(blocks, 64, self.hidden)], 1).reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], 0).contiguous()
        self.w_down = tensors[px + "down_proj.weight"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tiled and fused_epilogue(x):
            act = ops.skinny_gemm_swiglu(x, self.w_gate_up)
        elif self.tiled and dense_product(x, 2 * self.inter, "swiglu"):
            act = ops.dense_gemm_swiglu(x, self.w_gate_up)
        else:
            gate_up = project(x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            ops.silu_mul(act, gate_up, self.tiled)
        return last_product(act, self.w_down, self.defer_output)
