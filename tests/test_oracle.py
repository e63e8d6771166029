"""CPU: the oracle against its golden fixtures, against the independent numpy restatement, and
against closed-form cases.  The reference pins nothing for this path (no tests, no vectors), so
these are the pins the GPU parity tests stand on."""
import numpy as np
import pytest

import oracle
from oracle import numpy_restatement as nr
from tests.golden.make_golden import WORKLOADS, workload_image


@pytest.mark.parametrize("name", ["mandelbrot_1080p", "julia_512", "mandelbrot_ragged"])
def test_escape_matches_golden_digest(golden, name):
    img, total = workload_image(name)
    s, w = oracle.digest_u32(img)
    assert [s, w] == [int(v) for v in golden[f"{name}_digest"]]
    assert s == total
    if f"{name}_counts" in golden:
        assert np.array_equal(img, golden[f"{name}_counts"].astype(np.uint32))
    else:
        rows = golden[f"{name}_rows"]
        assert np.array_equal(img[rows], golden[f"{name}_row_counts"].astype(np.uint32))


def test_escape_julia_16k_rows_match_golden(golden):
    kind, W, H, x0, x1, y0, y1, cr, ci, mi = WORKLOADS["julia_16k"]
    dx, dy = oracle.grid_steps(x0, x1, y0, y1, W, H)
    rows = golden["julia_16k_rows"]
    for k, r in enumerate(rows):
        img, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, cr, ci, mi, row_begin=int(r), row_step=1, row_count=1)
        assert np.array_equal(img[0], golden["julia_16k_row_counts"][k].astype(np.uint32))


@pytest.mark.parametrize("name,stride", [("mandelbrot_1080p", 37), ("julia_512", 5), ("mandelbrot_ragged", 1)])
def test_escape_c_equals_numpy_restatement(name, stride):
    kind, W, H, x0, x1, y0, y1, cr, ci, mi = WORKLOADS[name]
    dx, dy = oracle.grid_steps(x0, x1, y0, y1, W, H)
    rows = np.arange(0, H, stride)
    c_img, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, cr, ci, mi, row_begin=0, row_step=stride)
    n_img = nr.escape_time(kind, W, H, x0, y0, dx, dy, cr, ci, mi, rows=rows)
    assert np.array_equal(c_img, n_img)


def test_escape_closed_form_points():
    # c = 0 never escapes; |c| > 2 escapes after exactly one update (test-before-update rule:
    # z0 = 0 passes the first test, z1 = c fails the second), fractal.py:21-24.
    one = lambda x, y, mi=50: int(oracle.escape_time(oracle.MANDELBROT, 1, 1, x, y, 0.0, 0.0, max_iter=mi)[0][0, 0])
    assert one(0.0, 0.0) == 50
    assert one(3.0, 0.0) == 1
    assert one(0.0, -2.5) == 1
    assert one(-1.0, 0.0) == 50          # period-2 point of the set
    assert one(0.25, 0.0, 1000) == 1000  # cusp, in the set
    assert one(0.0, 0.0, 0) == 0         # max_iter = 0: no update is ever made
    # Julia: a start outside radius 2 fails the very first test
    j = oracle.escape_time(oracle.JULIA, 1, 1, 2.5, 0.0, 0.0, 0.0, cr=-0.8, ci=0.156, max_iter=100)[0]
    assert int(j[0, 0]) == 0


def test_escape_norm_test_and_colour_follow_fractal_py():
    # fractal.py:22 `while z.norm() < 20 and iterations < 50`, :25 colour = 1 - iterations*0.02
    n = 16
    dx = np.float32(2.0 / n)
    img, _ = oracle.escape_time(oracle.JULIA, 2 * n, n, -2.0, -1.0, dx, dx, cr=-0.8, ci=0.2, max_iter=50,
                                test=oracle.TEST_NORM_GE, bound=20.0)
    ref = nr.escape_time(1, 2 * n, n, -2.0, -1.0, dx, dx, cr=-0.8, ci=0.2, max_iter=50, test=1, bound=20.0)
    assert np.array_equal(img, ref)
    col = oracle.escape_color(img, 0.02)
    assert np.array_equal(col, (np.float32(1.0) - img.astype(np.float32) * np.float32(0.02)).astype(np.float32))
    assert col.min() >= -1e-6 and col.max() <= 1.0


def test_float_ops_match_golden_and_numpy(golden):
    out = oracle.fused_map(golden["map_a"], golden["map_x"], golden["map_y"])
    assert np.array_equal(out, golden["map_out"])
    assert oracle.ulp_diff(nr.fused_map(golden["map_a"], golden["map_x"], golden["map_y"]), out).max() <= 1
    m = golden["rows_in"]
    assert np.array_equal(oracle.row_sum(m), golden["rows_sum"])
    assert np.array_equal(oracle.row_max(m), golden["rows_max"])
    assert np.array_equal(oracle.row_softmax(m), golden["rows_softmax"])
    assert oracle.ulp_diff(nr.row_softmax(m), golden["rows_softmax"]).max() <= 1
    assert np.allclose(oracle.row_softmax(m).astype(np.float64).sum(axis=1), 1.0, atol=1e-6)
    assert np.allclose(oracle.col_sum(m), m.astype(np.float64).sum(axis=0), rtol=1e-6)


def test_mse_matches_golden_numpy_and_finite_differences(golden):
    W, x, b, t = golden["mse_W"], golden["mse_x"], golden["mse_b"], golden["mse_t"]
    loss = oracle.mse_tanh_fwd(W, x, b, t)
    dW, dx, db = oracle.mse_tanh_bwd(W, x, b, t)
    assert loss == pytest.approx(float(golden["mse_loss"][0]), rel=1e-14)
    assert np.array_equal(dW, golden["mse_dW"]) and np.array_equal(dx, golden["mse_dx"])
    assert np.allclose(db, golden["mse_db"], rtol=1e-13, atol=0)
    nl, ndW, ndx, ndb = nr.mse_tanh(W, x, b, t)
    assert loss == pytest.approx(nl, rel=1e-12)
    assert np.allclose(dW, ndW, rtol=1e-6, atol=1e-12) and np.allclose(dx, ndx, rtol=1e-6, atol=1e-12)
    assert np.allclose(db, ndb, rtol=1e-10)
    # central finite differences in binary64 on a few coordinates
    f = lambda W_, b_: nr.mse_tanh(W_, x, b_, t)[0]
    eps = 1e-3
    for (r, c) in [(0, 0), (5, 17), (12, 35)]:
        Wp, Wm = W.astype(np.float64).copy(), W.astype(np.float64).copy()
        Wp[r, c] += eps
        Wm[r, c] -= eps
        # numpy restatement promotes float32 inputs; feed float64 perturbed copies through its formula directly
        y = lambda Wv: (np.tanh(Wv * x.astype(np.float64) + b.astype(np.float64)[None, :]) - t.astype(np.float64))
        fd = ((y(Wp) ** 2).sum() - (y(Wm) ** 2).sum()) / W.size / (2 * eps)
        assert fd == pytest.approx(float(ndW[r, c]), rel=1e-4, abs=1e-9)
    bp, bm = b.astype(np.float64).copy(), b.astype(np.float64).copy()
    bp[3] += eps
    bm[3] -= eps
    yb = lambda bv: (np.tanh(W.astype(np.float64) * x.astype(np.float64) + bv[None, :]) - t.astype(np.float64))
    fd = ((yb(bp) ** 2).sum() - (yb(bm) ** 2).sum()) / W.size / (2 * eps)
    assert fd == pytest.approx(float(ndb[3]), rel=1e-4)
    del f


def test_row_sharded_loss_adds_up(golden):
    W, x, b, t = golden["mse_W"], golden["mse_x"], golden["mse_b"], golden["mse_t"]
    denom = W.size
    parts = [oracle.mse_tanh_fwd(W[:6], x[:6], b, t[:6], denom), oracle.mse_tanh_fwd(W[6:], x[6:], b, t[6:], denom)]
    assert sum(parts) == pytest.approx(oracle.mse_tanh_fwd(W, x, b, t), rel=1e-13)


def test_coordinate_folding_of_the_front_end_differs_from_fractal_py_on_a_known_few_pixels():
    """fractal.py:20 computes a pixel's coordinate as ((i / n - 1) * 2, (j / n - 0.5) * 2), operation by
    operation in binary32; the front end (vernondsl_b200.lang) folds that affine expression exactly and
    the device computes origin + float(i) * step with origin and step rounded once.  The two agree as
    real numbers and differ in the last bits of some coordinates; this pins how far that reaches for the
    reference's own frame (n = 320): a sixth of the coordinates, and a handful of boundary pixels per
    frame.  It is a documented departure (the reference's runtime cannot be run here to say which
    rounding its generated shader really performs)."""
    f = np.float32
    n = 320
    i, j = np.arange(2 * n, dtype=np.float32), np.arange(n, dtype=np.float32)
    xa, ya = ((i / f(n)) - f(1)) * f(2), ((j / f(n)) - f(0.5)) * f(2)
    step = f(2.0 / n)
    xb, yb = f(-2.0) + i * step, f(-1.0) + j * step
    assert np.abs(xa.astype(np.float64) - xb).max() <= 2.0 ** -21 and np.abs(ya.astype(np.float64) - yb).max() <= 2.0 ** -21
    assert 0 < int((xa != xb).sum()) <= 2 * n // 4 and int((ya != yb).sum()) <= n // 4

    def counts(x, y, ci):
        zr = np.repeat(x[:, None], y.size, 1).astype(np.float32)
        zi = np.repeat(y[None, :], x.size, 0).astype(np.float32)
        cnt, live = np.zeros(zr.shape, np.int32), np.ones(zr.shape, bool)
        for _ in range(50):
            a, b = zr * zr, zi * zi
            live &= np.sqrt(a + b) < f(20)
            t = zr * zi
            zr, zi = np.where(live, (a - b) + f(-0.8), zr), np.where(live, (t + t) + f(ci), zi)
            cnt += live
        return cnt

    ci = f(np.cos(f(0.3))) * f(0.2)
    differing = int((counts(xa, ya, ci) != counts(xb, yb, ci)).sum())
    assert differing <= 2 * n * n // 10000   # at most 0.01 % of the frame's pixels


@pytest.mark.parametrize("bound", [4.0, 6.25, 400.0, 1.0e30])
def test_escape_is_final_in_binary32_where_blocks_of_updates_run_untested(bound):
    """The premise of the kernel that runs blocks of updates without a test (vernondsl_b200/csrc/k_escape_pair.cu):
    for bound >= 4 and |c| <= 1.5, once a + b > bound the test `!(a + b <= bound)` stays true on every later step,
    in the exact binary32 operation order of the loop (fractal.py:11-13,22-24), through overflow to Inf and NaN.
    One test after a block therefore says whether any step inside the block would have ended the pixel."""
    f = np.float32
    rng = np.random.default_rng(17)
    n = 400_000
    # starting points just outside the bound, a little further out, and far out (overflow within a few steps)
    radius = np.sqrt(np.float64(bound)) * np.concatenate([1.0 + rng.uniform(0, 1e-6, n // 4), 1.0 + rng.uniform(0, 1e-2, n // 4),
                                                         rng.uniform(1.0, 4.0, n // 4), 10.0 ** rng.uniform(0, 12, n // 4)])
    angle = rng.uniform(0, 2 * np.pi, n)
    zr, zi = (radius * np.cos(angle)).astype(f), (radius * np.sin(angle)).astype(f)
    cabs = np.where(rng.uniform(size=n) < 0.25, 1.5, rng.uniform(0, 1.5, n))      # a quarter on the limit |c| = 1.5 itself
    cang = rng.uniform(0, 2 * np.pi, n)
    cr, ci = (cabs * np.cos(cang)).astype(f), (cabs * np.sin(cang)).astype(f)
    inside_limit = cr.astype(np.float64) ** 2 + ci.astype(np.float64) ** 2 <= 2.25   # the launcher's own condition on c
    b32 = f(min(bound, 3.0e38))
    with np.errstate(over="ignore", invalid="ignore"):
        a, b = zr * zr, zi * zi
        started = ~((a + b) <= b32) & inside_limit
        assert started.sum() > n // 2
        for step in range(30):
            t = zr * zi
            zi = (t + t) + ci
            zr = (a - b) + cr
            a, b = zr * zr, zi * zi
            still = ~((a + b) <= b32)
            assert still[started].all(), (bound, step, int((~still[started]).sum()))


def test_below_the_limits_of_the_untested_blocks_escape_is_not_final():
    """Why the launcher sends bound < 4 to the kernel that tests every step: with |c| = 1.5 and bound 3, points just
    outside the bound come back inside it (the condition bound >= 4 is not slack)."""
    f = np.float32
    rng = np.random.default_rng(17)
    n = 100_000
    radius = np.sqrt(3.0) * (1.0 + rng.uniform(0, 1e-2, n))
    angle, cang = rng.uniform(0, 2 * np.pi, n), rng.uniform(0, 2 * np.pi, n)
    zr, zi = (radius * np.cos(angle)).astype(f), (radius * np.sin(angle)).astype(f)
    cr, ci = (1.5 * np.cos(cang)).astype(f), (1.5 * np.sin(cang)).astype(f)
    a, b = zr * zr, zi * zi
    t = zr * zi
    zi2, zr2 = (t + t) + ci, (a - b) + cr
    came_back = ((zr2 * zr2 + zi2 * zi2) <= f(3.0)) & ~((a + b) <= f(3.0))
    assert came_back.sum() > 100
