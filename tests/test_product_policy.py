"""Which of a layer's products go to which kernel (kernels/gemm.py): decided on the host from sizes alone."""

import pytest
import torch

from dli_b200.kernels import gemm


class Shape:
    """What the policy looks at of its activations."""

    def __init__(self, tokens, width, dtype=torch.bfloat16):
        self.shape, self.dtype = (tokens, width), dtype


def test_few_tokens_go_to_the_decode_product_and_its_epilogues():
    assert gemm.fused_epilogue(Shape(1, 2048)) and gemm.fused_epilogue(Shape(8, 2048))
    assert not gemm.fused_epilogue(Shape(9, 2048))
    assert not gemm.fused_epilogue(Shape(4, 2048, torch.float32))  # the float32 path stays with true 32-bit products
    assert gemm.decode_product(Shape(64, 2048), gemm.SKINNY_MAX_TOKENS_HEAD) and not gemm.decode_product(Shape(65, 2048), gemm.SKINNY_MAX_TOKENS_HEAD)


def test_long_portions_take_the_many_token_product_for_gate_up():
    for tokens in (512, 2048, 8192, 100000):
        assert gemm.dense_product(Shape(tokens, 2048), 16384, "swiglu")
    assert not gemm.dense_product(Shape(511, 2048), 16384, "swiglu")
    assert not gemm.dense_product(Shape(2048, 2048, torch.float32), 16384, "swiglu")
    assert not gemm.dense_product(Shape(2048, 2044), 16384, "swiglu")  # K must be a multiple of 8 (16-byte rows for TMA)
    with pytest.raises(ValueError):
        gemm.dense_product(Shape(2048, 2048), 2048, "residual")


def test_q_k_v_takes_it_when_its_tiles_fill_their_rounds():
    """74 pairs of SMs (148 without a device): 3,072 features are 12 tiles wide."""
    assert gemm.dense_product(Shape(512, 2048), 3072, "rotary")  # 24 tiles: one round
    assert gemm.dense_product(Shape(1024, 2048), 3072, "rotary")  # 48 tiles: one round
    assert not gemm.dense_product(Shape(2048, 2048), 3072, "rotary")  # 96 tiles: two rounds, the second 30 % full
    assert gemm.dense_product(Shape(4096, 2048), 3072, "rotary")  # 192 of 222
    assert gemm.dense_product(Shape(8192, 2048), 3072, "rotary")  # 384 of 444
