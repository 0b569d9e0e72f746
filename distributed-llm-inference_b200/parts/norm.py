"""RMS normalisation, fused with the residual addition that precedes it."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = (h + delta) * rsqrt(mean((h + delta)^2) + eps) * weight, all in float32 and rounded
    once (src/dli/model/llama.py:41-44 rounds before the weight product; one rounding is closer
    to the float32 result).  params: size, eps."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.spec.prefix + "weight": TensorDecl((self.size,), "vector32")}

    def load(self, tensors):
        self.weight = tensors[self.spec.prefix + "weight"]

    def add_norm(self, h: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        y = torch.empty((n, self.size), dtype=self.env.dtype, device=h.device)
        ops.add_rmsnorm(y, h, delta, self.weight, self.eps, rows)
        return y

    def add_product_norm(self, h: torch.Tensor, product) -> ops.ScaledRows | None:
        """h += product (computed here, float32 sums added to float32 h) and the norm's first half
        in the product's epilogue; the factor rsqrt(mean(h^2) + eps) of each row travels with the
        result and is applied by the product that reads it, to its float32 sums."""
        if not ops.skinny_gemm_supported(h.shape[0], self.size) or h.shape[0] > 64:
            return None  # the product that reads the result could not take rows of this size
        return ops.skinny_gemm_residual(product.x, product.weight, h, self.weight, self.eps)
