"""GPU: tanh-MSE loss and its hand-fused backward against the binary64 CPU oracle."""
import numpy as np
import pytest

import oracle
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu
RTOL = 1e-5  # gradients and loss: relative error, norm-wise (against the largest magnitude of the reference array)


def problem(rows, cols, seed=3001):
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    return f(rows, cols), f(rows, cols), f(cols), f(rows, cols)


def normwise(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got.astype(np.float64) - want).max() / max(np.abs(want).max(), 1e-300))


def run_bwd(dev, stream, W, x, b, t, denom=0.0, with_loss=True):
    rows, cols = W.shape
    bufs = [dev.from_numpy(v) for v in (W, x, b, t)]
    dW, dx, db = dev.empty((rows, cols), np.float32), dev.empty((rows, cols), np.float32), dev.empty(cols, np.float32)
    loss = dev.empty(1, np.float32) if with_loss else None
    ops.mse_tanh_bwd(stream, *bufs, dW, dx, db, rows, cols, denom, loss)
    stream.check()
    out = dW.download(), dx.download(), db.download(), (loss.download()[0] if with_loss else None)
    for bf in bufs + [dW, dx, db] + ([loss] if with_loss else []):
        bf.close()
    return out


@pytest.mark.parametrize("rows,cols", [(13, 36), (64, 4096), (1000, 1024), (3, 5), (1, 1), (257, 1028), (50, 1001)])
def test_backward_matches_oracle(dev, stream, rows, cols):
    W, x, b, t = problem(rows, cols)
    dW, dx, db, loss = run_bwd(dev, stream, W, x, b, t)
    rW, rx, rb = oracle.mse_tanh_bwd(W, x, b, t)
    assert normwise(dW, rW) <= RTOL and normwise(dx, rx) <= RTOL and normwise(db, rb) <= RTOL
    assert loss == pytest.approx(oracle.mse_tanh_fwd(W, x, b, t), rel=RTOL)
    # elementwise, away from the cancellation y ~ t, the relative error is small too
    big = np.abs(rW) > 1e-3 * np.abs(rW).max()
    assert (np.abs(dW[big] - rW[big]) <= 1e-4 * np.abs(rW[big])).all()


def test_forward_matches_oracle(dev, stream):
    for rows, cols in [(13, 36), (512, 4096), (77, 1001)]:
        W, x, b, t = problem(rows, cols, seed=5)
        bufs = [dev.from_numpy(v) for v in (W, x, b, t)]
        loss = dev.empty(1, np.float32)
        ops.mse_tanh_fwd(stream, *bufs, loss, rows, cols)
        stream.check()
        assert loss.download()[0] == pytest.approx(oracle.mse_tanh_fwd(W, x, b, t), rel=RTOL)


def test_golden(dev, stream, golden):
    W, x, b, t = golden["mse_W"], golden["mse_x"], golden["mse_b"], golden["mse_t"]
    dW, dx, db, loss = run_bwd(dev, stream, W, x, b, t)
    assert normwise(dW, golden["mse_dW"]) <= RTOL and normwise(dx, golden["mse_dx"]) <= RTOL
    assert normwise(db, golden["mse_db"]) <= RTOL
    assert loss == pytest.approx(float(golden["mse_loss"][0]), rel=RTOL)


def test_saturated_tanh_keeps_relative_accuracy(dev, stream):
    # |W*x + b| up to ~9: 1 - tanh^2 is ~1e-7 there; the 4E/(1+E)^2 form must not lose it
    rows, cols = 32, 256
    rng = np.random.default_rng(8)
    W = rng.uniform(2.0, 3.0, (rows, cols)).astype(np.float32)
    x = rng.uniform(2.0, 3.0, (rows, cols)).astype(np.float32)
    b = np.zeros(cols, np.float32)
    t = np.zeros((rows, cols), np.float32)
    dW, dx, db, _ = run_bwd(dev, stream, W, x, b, t)
    rW, rx, rb = oracle.mse_tanh_bwd(W, x, b, t)
    assert np.allclose(dW, rW, rtol=1e-5, atol=0) and np.allclose(dx, rx, rtol=1e-5, atol=0)
    assert np.allclose(db, rb, rtol=1e-5, atol=0)


def test_row_shards_add_up_to_the_whole(dev, stream):
    """Two row shards with the whole problem's denominator: dW/dx concatenate, db and loss add."""
    rows, cols = 96, 512
    W, x, b, t = problem(rows, cols, seed=11)
    full = run_bwd(dev, stream, W, x, b, t)
    denom = float(rows * cols)
    lo = run_bwd(dev, stream, W[:40], x[:40], b, t[:40], denom)
    hi = run_bwd(dev, stream, W[40:], x[40:], b, t[40:], denom)
    assert np.allclose(np.concatenate([lo[0], hi[0]]), full[0], rtol=1e-6, atol=1e-12)
    assert np.allclose(np.concatenate([lo[1], hi[1]]), full[1], rtol=1e-6, atol=1e-12)
    assert normwise(lo[2] + hi[2], full[2].astype(np.float64)) <= RTOL
    assert lo[3] + hi[3] == pytest.approx(full[3], rel=RTOL)


def test_bit_reproducible(dev, stream):
    W, x, b, t = problem(2048, 4096, seed=2)
    a = run_bwd(dev, stream, W, x, b, t)
    c = run_bwd(dev, stream, W, x, b, t)
    assert all(np.array_equal(p, q) for p, q in zip(a[:3], c[:3])) and a[3] == c[3]


def test_errors(dev, stream):
    W, x, b, t = problem(8, 16)
    bufs = [dev.from_numpy(v) for v in (W, x, b, t)]
    dW, dx, db = dev.empty((8, 16), np.float32), dev.empty((8, 16), np.float32), dev.empty(8, np.float32)  # db too small
    with pytest.raises(L.VrhiError) as e:
        ops.mse_tanh_bwd(stream, *bufs, dW, dx, db, 8, 16)
    assert e.value.status == L.ERR_SIZE
    with pytest.raises(L.VrhiError) as e:
        ops.launch(stream, "mse_tanh_bwd", [bf.arg(L.INPUT) for bf in bufs], ops._mse(8, 16, 0))
    assert e.value.status == L.ERR_INVALID
