"""GPU: row sum / max / softmax and column sums against the binary64 CPU oracle (1e-5 relative)."""
import numpy as np
import pytest

import oracle
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu
RTOL = 1e-5  # relative tolerance for reductions and softmax


def matrix(rows, cols, seed=2001):
    return (2.0 * np.random.default_rng(seed).standard_normal((rows, cols))).astype(np.float32)  # N(0, 4): sigma = 2


SHAPES = [(1, 4), (3, 128), (257, 4096), (9, 260), (5, 4092), (33, 1000), (4, 8192), (7, 13), (2, 1), (1000, 36), (3, 5000)]


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_row_ops_match_oracle(dev, stream, rows, cols):
    m = matrix(rows, cols)
    M = dev.from_numpy(m)
    s, mx, sm = dev.empty(rows, np.float32), dev.empty(rows, np.float32), dev.empty((rows, cols), np.float32)
    ops.row_sum(stream, M, s, rows, cols)
    ops.row_max(stream, M, mx, rows, cols)
    ops.row_softmax(stream, M, sm, rows, cols)
    stream.check()
    want_sum = oracle.row_sum(m)
    scale = np.abs(m).astype(np.float64).sum(axis=1)  # a sum of signed terms: error relative to the sum of magnitudes
    assert (np.abs(s.download() - want_sum) <= RTOL * scale + 1e-30).all()
    assert np.array_equal(mx.download(), oracle.row_max(m))
    got = sm.download()
    want = oracle.row_softmax(m)
    assert np.allclose(got, want, rtol=RTOL, atol=1e-38)
    assert np.allclose(got.astype(np.float64).sum(axis=1), 1.0, atol=1e-5)
    # fused variant gives the same three results from one read
    s2, mx2, sm2 = dev.empty(rows, np.float32), dev.empty(rows, np.float32), dev.empty((rows, cols), np.float32)
    ops.row_stats_softmax(stream, M, s2, mx2, sm2, rows, cols)
    stream.check()
    # (the one-pass kernel groups the row differently across warps, so its sum may round differently)
    assert (np.abs(s2.download() - want_sum) <= RTOL * scale + 1e-30).all()
    assert np.array_equal(mx2.download(), mx.download())
    assert np.array_equal(sm2.download(), got)
    for b in (M, s, mx, sm, s2, mx2, sm2):
        b.close()


def test_row_ops_golden(dev, stream, golden):
    m = golden["rows_in"]
    rows, cols = m.shape
    M = dev.from_numpy(m)
    s, mx, sm = dev.empty(rows, np.float32), dev.empty(rows, np.float32), dev.empty((rows, cols), np.float32)
    ops.row_stats_softmax(stream, M, s, mx, sm, rows, cols)
    stream.check()
    assert np.allclose(s.download(), golden["rows_sum"], rtol=RTOL, atol=1e-4)
    assert np.array_equal(mx.download(), golden["rows_max"])
    assert np.allclose(sm.download(), golden["rows_softmax"], rtol=RTOL, atol=1e-38)


def test_softmax_is_shift_invariant_and_stable(dev, stream):
    rows, cols = 64, 4096
    m = matrix(rows, cols, seed=5)
    big = (m + np.float32(1000.0)).astype(np.float32)   # exp(1000) overflows without the max subtraction
    M, B = dev.from_numpy(m), dev.from_numpy(big)
    a, b = dev.empty((rows, cols), np.float32), dev.empty((rows, cols), np.float32)
    ops.row_softmax(stream, M, a, rows, cols)
    ops.row_softmax(stream, B, b, rows, cols)
    stream.check()
    ga, gb = a.download(), b.download()
    assert np.isfinite(gb).all()
    assert np.allclose(gb, oracle.row_softmax(big), rtol=RTOL, atol=1e-38)
    assert np.allclose(ga, oracle.row_softmax(m), rtol=RTOL, atol=1e-38)


def test_reductions_are_bit_reproducible(dev, stream):
    rows, cols = 4096, 4096
    m = matrix(rows, cols, seed=9)
    M = dev.from_numpy(m)
    outs = []
    for _ in range(3):
        s, c = dev.empty(rows, np.float32), dev.empty(cols, np.float32)
        ops.row_sum(stream, M, s, rows, cols)
        ops.col_sum(stream, M, c, rows, cols)
        stream.check()
        outs.append((s.download(), c.download()))
    for s, c in outs[1:]:
        assert np.array_equal(s, outs[0][0]) and np.array_equal(c, outs[0][1])


@pytest.mark.parametrize("rows,cols", [(1, 4), (300, 4096), (17, 1001), (5000, 12), (2, 3)])
def test_col_sum_matches_oracle(dev, stream, rows, cols):
    m = matrix(rows, cols, seed=4)
    M = dev.from_numpy(m)
    c = dev.empty(cols, np.float32)
    ops.col_sum(stream, M, c, rows, cols)
    stream.check()
    scale = np.abs(m).astype(np.float64).sum(axis=0)
    assert (np.abs(c.download() - oracle.col_sum(m)) <= RTOL * scale + 1e-30).all()


def test_rows_errors_and_empty(dev, stream):
    M = dev.from_numpy(np.zeros((8, 8), np.float32))
    small = dev.empty(2, np.float32)  # allocations are at least 16 bytes: room for 4 row results, not 8
    with pytest.raises(L.VrhiError) as e:
        ops.row_sum(stream, M, small, 8, 8)
    assert e.value.status == L.ERR_SIZE and "argument 1" in e.value.message
    with pytest.raises(L.VrhiError) as e:
        ops.row_sum(stream, M, small, 16, 8)  # input too small for the declared shape
    assert e.value.status == L.ERR_SIZE and "input" in e.value.message
    ops.row_sum(stream, M, small, 0, 8)  # zero rows: nothing to do, not an error
    stream.check()
