"""SwiGLU feed-forward."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.gemm import project
from ..weights.loader import TensorDecl
from .base import Part, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)) (src/dli/model/llama.py:189-191).  gate and up are read by
    their own names and stacked at load, so one product yields gate | up.
    params: hidden_size, intermediate_size."""

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up: torch.Tensor | None = None
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
        self.w_gate_up = torch.cat([tensors[px + "gate_proj.weight"], tensors[px + "up_proj.weight"]], 0).contiguous()
        self.w_down = tensors[px + "down_proj.weight"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate_up = project(x, self.w_gate_up)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.silu_mul(act, gate_up)
        return project(act, self.w_down)
