"""fl_gemm_tc_static_scratch, the entry point for callers that cannot allocate.

Some users of the compiled library have no device allocator to call: all of the
GPU's memory already belongs to a pool of their own, or they run where the CUDA
allocation calls are off limits or would stall work in flight.  The split-K
product needs a float workspace, so for them the library carries one inside
itself (8 MiB per GPU) and exposes this one C symbol that uses it.

The test calls the symbol through ctypes, exactly as such a user would, twice in
a row with different problems (the second smaller, so that what the first left
in the shared array lies beside it), and compares each result with the ordinary
entry point's (fl_gemm_tc, given a workspace) within the tolerance of the other
GEMM tests.  It also checks that a problem beyond the array is refused with a
message and launches nothing.

The file's name makes pytest collect it last: a run that stops at the first
failure has then already run every other test.
"""
import ctypes
import math
from ctypes import c_char_p, c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 21
ERR_TOO_SMALL = -2


def entry_point():
    from fastllm_py_b200.native.build import load_library

    lib = load_library("gemm_tcgen05")
    fn = lib.fl_gemm_tc_static_scratch
    fn.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_int, c_int,
                   c_int, c_int, c_int, c_void_p, c_void_p, c_char_p, c_int]
    fn.restype = c_int
    return fn


def call(fn, a, w, out, bn, splits, status):
    text = ctypes.create_string_buffer(512)
    rc = fn(c_void_p(a.data_ptr()), a.stride(0), c_void_p(w.data_ptr()), w.stride(0),
            c_void_p(out.data_ptr()), 0 if out.dtype == torch.float32 else 1, out.stride(0),
            a.shape[0], w.shape[0], a.shape[1], bn, splits,
            torch.cuda.get_device_properties(0).multi_processor_count,
            c_void_p(status.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream), text, 512)
    return rc, text.value.decode()


def problem(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    return a, w


def test_two_calls_match_the_ordinary_entry_point():
    from fastllm_py_b200.native import gemm_tc

    fn = entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # (m, n, k, bn, splits, out dtype): the second problem is smaller than the first; the third lets
    # the library plan (bn = 0; a few tokens of a narrow product: it splits K); the fourth is the
    # CTA-pair kernel (code 512: tiles of 256 tokens) with K split, which still fits the array
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert gemm_tc.plan(8, 256, 2048, sms)[1] > 1
    assert 3 * 300 * 512 <= SCRATCH_FLOATS
    for seed, (m, n, k, bn, splits, dt) in enumerate([(48, 640, 1024, 64, 4, torch.float32),
                                                       (5, 200, 520, 16, 3, torch.bfloat16),
                                                       (8, 256, 2048, 0, 0, torch.bfloat16),
                                                       (300, 512, 1600, 512, 3, torch.float32)]):
        a, w = problem(m, n, k, seed)
        got = torch.full((m, n), float("nan"), dtype=dt, device=DEV)
        rc, text = call(fn, a, w, got, bn, splits, status)
        assert rc == 0, f"entry point returned {rc}: {text}"
        want = torch.zeros((m, n), dtype=dt, device=DEV)
        gemm_tc.gemm(a, w, want, bn=bn, splits=splits)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        exact = a.float() @ w.float().t()
        tol = 1e-3 * math.sqrt(k) if dt == torch.float32 else 2 ** -8 * float(exact.abs().max()) + 1e-3
        assert float((got.float() - want.float()).abs().max()) <= tol
        assert float((got.float() - exact).abs().max()) <= tol


def test_a_problem_beyond_the_array_is_refused():
    fn = entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    m, n, k, splits = 64, 8192 + 64, 512, 8            # 8 * 64 * 8256 floats > 2 Mi
    assert splits * m * n > SCRATCH_FLOATS
    a, w = problem(m, n, k, 3)
    out = torch.full((m, n), 7.0, dtype=torch.float32, device=DEV)
    rc, text = call(fn, a, w, out, 64, splits, status)
    torch.cuda.synchronize()
    assert rc == ERR_TOO_SMALL
    assert str(splits * m * n) in text and str(SCRATCH_FLOATS) in text
    assert bool(torch.all(out == 7.0)), "a refused call must not launch anything"
    # a tile width without a split count is the caller's mistake, as it is for fl_gemm_tc
    rc, _ = call(fn, a, w, out, 64, 0, status)
    assert rc == 1                                       # cudaErrorInvalidValue
    assert bool(torch.all(out == 7.0))
