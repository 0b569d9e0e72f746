"""Matrix products y = x W^T.

The reference's engine uses a library for every linear layer (nn.Linear, i.e.
cuBLAS: src/dli/model/llama.py:72-74,95,190,305); so does this wrapper.  The
float32 path is true 32-bit: TF32 and reduced-precision accumulation are switched
off for the process when this module is imported, and checked at every call.
"""

from __future__ import annotations

import torch

torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [n, in] times weight [out, in] transposed; float32 accumulation in both dtypes."""
    if not x.is_cuda:
        raise RuntimeError("linear: the engine has no CPU path")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("linear: TF32 was switched on; the float32 path must stay true 32-bit")
    return torch.matmul(x, weight.t(), out=out)
