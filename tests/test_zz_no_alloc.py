"""GPU: the allocation-free column-sum entry point (vrhi_col_sum_static_scratch).

It serves callers that cannot allocate at call time -- latency-bound frame or control loops,
processes whose device memory was divided between tenants up front -- by keeping its partial sums
in a fixed array inside the library instead of the stream arena.  The test calls it through the
C ABI with raw device pointers, twice in a row on different data (the array keeps the first
call's contents, which the second call must not see), and compares with the existing "col_sum"
operator within the tolerance the reduction tests use.

This file is named to be collected last: a run that stops at the first failure has by then run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu
RTOL = 1e-5  # as in test_rows_gpu.py: relative to the sum of magnitudes of each column


def static_col_sum(in_buf, out_buf, rows, cols, cuda_stream=None):
    return L.lib().vrhi_col_sum_static_scratch(C.c_void_p(in_buf.ptr), C.c_void_p(out_buf.ptr), rows, cols,
                                               C.c_void_p(cuda_stream) if cuda_stream else None)


@pytest.mark.parametrize("rows,cols", [(300, 4096), (1000, 1001), (5, 12), (4096, 64)])
def test_matches_col_sum_on_two_calls_in_a_row(dev, stream, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    for call in range(2):
        m = (2.0 * rng.standard_normal((rows, cols)) + call).astype(np.float32)
        M = dev.from_numpy(m)
        want_buf, got_buf = dev.empty(cols, np.float32), dev.empty(cols, np.float32)
        got_buf.fill(0xEE)
        ops.col_sum(stream, M, want_buf, rows, cols)
        stream.check()
        assert static_col_sum(M, got_buf, rows, cols) == L.OK   # default stream
        dev.synchronize()
        want, got = want_buf.download(), got_buf.download()
        scale = np.abs(m).astype(np.float64).sum(axis=0)
        assert (np.abs(got.astype(np.float64) - want) <= RTOL * scale + 1e-30).all()
        assert (np.abs(got.astype(np.float64) - oracle.col_sum(m)) <= RTOL * scale + 1e-30).all()
        for b in (M, want_buf, got_buf):
            b.close()


def test_runs_on_a_callers_stream_without_touching_the_allocator(dev):
    import torch

    rows, cols = 2048, 4096
    m = torch.randn(rows, cols, device="cuda:0")
    out = torch.empty(cols, device="cuda:0")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    # first use on this device: CUDA loads the kernels' code and the entry point looks up its array
    assert L.lib().vrhi_col_sum_static_scratch(C.c_void_p(m.data_ptr()), C.c_void_p(out.data_ptr()), 8, cols, None) == L.OK
    torch.cuda.synchronize()
    held_before = dev.allocated()
    free_before, _ = torch.cuda.mem_get_info()
    rc = L.lib().vrhi_col_sum_static_scratch(C.c_void_p(m.data_ptr()), C.c_void_p(out.data_ptr()), rows, cols,
                                             C.c_void_p(s.cuda_stream))
    assert rc == L.OK
    s.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert dev.allocated() == held_before and free_after == free_before
    ref = m.double().sum(dim=0)
    scale = m.double().abs().sum(dim=0)
    assert bool(((out.double() - ref).abs() <= RTOL * scale).all())


def test_rejects_what_does_not_fit(dev):
    small = dev.empty(16, np.float32)
    rc = L.lib().vrhi_col_sum_static_scratch(C.c_void_p(small.ptr), C.c_void_p(small.ptr), 1, 262145, None)
    assert rc == L.ERR_SIZE and b"exceed the fixed scratch" in L.lib().vrhi_last_error()
    assert L.lib().vrhi_col_sum_static_scratch(None, C.c_void_p(small.ptr), 1, 4, None) == L.ERR_INVALID
    assert L.lib().vrhi_col_sum_static_scratch(C.c_void_p(small.ptr + 4), C.c_void_p(small.ptr), 1, 4, None) == L.ERR_SIZE
    small.close()
