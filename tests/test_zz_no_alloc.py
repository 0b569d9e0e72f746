"""The entry point that allocates nothing (csrc/no_alloc_entry.h), called through its exported C
symbol as an embedder would, against the ordinary entry point.

Some hosts of this library cannot call cudaMalloc once they run (their memory is planned up
front, or an allocation would stall their streams); for them the split-key decode attention has
a variant whose scratch is a fixed array inside the library.  The test runs it twice in a row
with different inputs (the array keeps the first call's contents) and checks that a request
beyond the array's size is refused.  It is collected last on purpose, and passes alone too.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SEQS = [(700, 1), (63, 1), (1500, 1), (0, 1), (255, 1)]
NH, NKV, D, PAGE = 8, 2, 64, 16
SCRATCH_FLOATS = 1 << 20


def entry_point():
    from dli_b200.csrc.build import load_library

    lib = load_library("attention_mma.cu", {"HEAD_DIM": D})
    fn = lib.dli_paged_decode_attention_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_int, c_void_p]
    fn.restype = c_int
    return fn


def call(fn, t, out, splits, num_seqs=len(SEQS), seq0=0, first_row=0):
    ptr = lambda x: c_void_p(x.data_ptr())
    return fn(ptr(out), ptr(t["qkv"]), t["qkv"].shape[1], ptr(t["kp"]), ptr(t["vp"]), ptr(t["tables"]), t["tables"].shape[1],
              ptr(t["q_start"]), ptr(t["kv_len"]), seq0, num_seqs, first_row, NH, NKV, PAGE, 0, D**-0.5, splits,
              c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_equals_the_ordinary_one_twice_in_a_row():
    from dli_b200.kernels import ops
    from tests.test_kernels_gpu import attention_case, tol

    fn = entry_point()
    for seed, splits in ((1, 4), (2, 7)):  # the second call finds the first call's leftovers in the array
        t = attention_case(NH, NKV, D, PAGE, SEQS, torch.bfloat16, seed=seed)
        rows = len(SEQS) * NH
        want = torch.full((t["n"], NH * D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        scratch = (torch.empty(rows * splits * D, device="cuda:0"), torch.empty(rows * splits * 2, device="cuda:0"))
        ops.paged_attention_mma(want, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 0, len(SEQS), 1, 0, NH,
                                D**-0.5, None, splits, scratch)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()  # what torch's allocator handed out ...
        free_before, _ = torch.cuda.mem_get_info()  # ... and what the driver has left: a cudaMalloc inside the library would show here
        assert call(fn, t, got, splits) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if seed > 1:  # (the very first call may load the library's device image, the array included)
            assert torch.cuda.mem_get_info()[0] == free_before, "device memory was taken during the call"
        np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(), atol=tol(torch.bfloat16, 2))
        assert not torch.isnan(got).any()


def test_no_alloc_entry_point_on_sequences_that_do_not_start_at_row_0():
    """The last three sequences of the batch only (seq0 = 2): their rows start at first_row = 2, and so do their
    places in the array."""
    from dli_b200.kernels import ops
    from tests.test_kernels_gpu import attention_case, tol

    fn = entry_point()
    t = attention_case(NH, NKV, D, PAGE, SEQS, torch.bfloat16, seed=5)
    splits, rows = 5, len(SEQS) * NH
    want = torch.full((t["n"], NH * D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    scratch = (torch.empty(rows * splits * D, device="cuda:0"), torch.empty(rows * splits * 2, device="cuda:0"))
    ops.paged_attention_mma(want, t["qkv"], t["kp"], t["vp"], t["tables"], t["q_start"], t["kv_len"], 2, 3, 1, 2, NH, D**-0.5, None, splits, scratch)
    got = torch.full_like(want, float("nan"))
    assert call(fn, t, got, splits, num_seqs=3, seq0=2, first_row=2) == 0
    torch.cuda.synchronize()
    assert torch.isnan(got[:2]).all() and not torch.isnan(got[2:]).any(), "rows of other sequences were written, or its own were not"
    np.testing.assert_allclose(got[2:].float().cpu().numpy(), want[2:].float().cpu().numpy(), atol=tol(torch.bfloat16, 2))
    # the need counts the rows in front: (first_row + num_seqs) * heads * splits * (head size + 2) floats
    most = SCRATCH_FLOATS // ((2 + 3) * NH * (D + 2))
    assert call(fn, t, got, most + 1, num_seqs=3, seq0=2, first_row=2) == 1002


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    from tests.test_kernels_gpu import attention_case

    fn = entry_point()
    t = attention_case(NH, NKV, D, PAGE, SEQS, torch.bfloat16, seed=3)
    out = torch.zeros((t["n"], NH * D), dtype=torch.bfloat16, device="cuda:0")
    too_many = SCRATCH_FLOATS // (len(SEQS) * NH * (D + 2)) + 1
    assert call(fn, t, out, too_many) == 1002  # DLI_ERR_SCRATCH_TOO_SMALL, nothing was launched
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
    assert call(fn, t, out, 0) == 1001  # DLI_ERR_UNSUPPORTED
