"""Matrix products y = x W^T.

The reference's engine uses a library for every linear layer (nn.Linear, i.e.
cuBLAS: src/dli/model/llama.py:72-74,95,190,305); so does this wrapper.  The
float32 path is true 32-bit: TF32 and reduced-precision accumulation are switched
off for the process when this module is imported, and checked at every call.
"""

from __future__ import annotations

import torch

from . import ops
from .attention import sm_count

torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


# Up to this many tokens a layer's bfloat16 products go to the engine's own tcgen05 kernel, which
# there beats the library on three of the four shapes and fuses the next elementwise step;
# measured on B200 at Llama-3.2-1B sizes, the library's kernels win from about 12 tokens on.
# The head's product (float32 logits straight from the accumulator) stays with it up to 64.
SKINNY_MAX_TOKENS = 8
SKINNY_MAX_TOKENS_HEAD = 64


def decode_product(x: torch.Tensor, max_tokens: int = SKINNY_MAX_TOKENS) -> bool:
    """Whether a product with these activations goes to the engine's own decode kernel."""
    return x.dtype == torch.bfloat16 and x.shape[0] <= max_tokens and ops.skinny_gemm_supported(x.shape[0], x.shape[1])


# Up to this many tokens the decode product also finishes the next elementwise step (rotary and
# cache write, SiLU * up) in its epilogue; with more tokens per CTA the separate kernels, which
# spread that work over the whole GPU, are faster.
FUSED_EPILOGUE_MAX_TOKENS = 8


def fused_epilogue(x: torch.Tensor) -> bool:
    return decode_product(x) and x.shape[0] <= FUSED_EPILOGUE_MAX_TOKENS


# From this many tokens two of a layer's bfloat16 products go to the engine's tcgen05 product for many tokens, which
# does the elementwise step behind the product in its epilogue.  Measured on B200 at Llama-3.2-1B sizes (us, this
# product against the library's product plus the kernel it saves; 512 / 2,048 / 8,192 tokens): gate|up with SiLU * up
# 39/38, 102/116, 383/427: always.  q|k|v with rotary and cache write 26/37, 39/37, 87/98: when its tiles fill their
# waves (2,048 tokens are 96 tiles on 74 pairs of SMs).  The plain product takes 1.00 of the library's time for gate|up
# at 2,048 tokens, 0.96-1.07 for o and down, which stay with the library: with the residual addition and the norm's
# sums in the epilogue they were slower than the library's product and the norm kernel (the epilogue read and wrote
# the float32 residual a row per thread), so that epilogue was taken out again.
DENSE_MIN_TOKENS = 512
DENSE_TILE = (256, 256)  # tokens x features of a tile, which a pair of SMs computes
WAVE_FILL_MIN = 0.8


def _dense_tiles(tokens: int, features: int) -> int:
    return -(-tokens // DENSE_TILE[0]) * -(-features // DENSE_TILE[1])


def _dense_candidate(x, features: int) -> bool:
    return x.dtype == torch.bfloat16 and x.shape[0] >= DENSE_MIN_TOKENS and ops.dense_gemm_supported(x.shape[1], features)


def dense_product(x, features: int, epilogue: str) -> bool:
    """Whether the product of these activations with a [features, K] weight, followed by ``epilogue`` ("swiglu" or
    "rotary"), goes to the engine's product for many tokens."""
    if not _dense_candidate(x, features):
        return False
    tiles, pairs = _dense_tiles(x.shape[0], features), max(1, sm_count() // 2)
    if epilogue == "swiglu":
        return True
    if epilogue == "rotary":
        return tiles <= pairs or tiles / (-(-tiles // pairs) * pairs) >= WAVE_FILL_MIN
    raise ValueError(f"unknown epilogue {epilogue!r}")


def project(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None, max_tokens: int = SKINNY_MAX_TOKENS) -> torch.Tensor:
    """y = x W^T for a step's tokens, in x's dtype or in ``out_dtype`` (float32 for logits).  x may be
    ops.ScaledRows (rows that still lack their norm's factor): those only exist for token counts that
    the decode kernel serves, which applies the factor."""
    if isinstance(x, ops.ScaledRows) or decode_product(x, max_tokens):
        return ops.skinny_gemm(x, weight, out_dtype or x.dtype)
    y = linear(x, weight)
    return y if out_dtype in (None, y.dtype) else y.to(out_dtype)


def last_product(x: torch.Tensor, weight: torch.Tensor, defer: bool):
    """The product that ends a mixer or feed-forward: x W^T, or — if the part's owner allowed it and
    the decode kernel with its fused epilogues will serve these tokens — the product left
    uncomputed for the norm behind it (parts.base.PendingProduct)."""
    if defer and fused_epilogue(x):
        from ..parts.base import PendingProduct

        return PendingProduct(x, weight)
    return project(x, weight)


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [n, in] times weight [out, in] transposed; float32 accumulation in both dtypes."""
    if not x.is_cuda:
        raise RuntimeError("linear: the engine has no CPU path")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("linear: TF32 was switched on; the float32 path must stay true 32-bit")
    return torch.matmul(x, weight.t(), out=out)
