"""GPU: execution graph -- fusion plan, kernel selection and reverse-mode gradients -- against
numpy float64 evaluations of the same expressions and the CPU oracle."""
import numpy as np
import pytest

import oracle
from oracle import numpy_restatement as nr
from vernondsl_b200 import _lib as L
from vernondsl_b200.graph import Graph

pytestmark = pytest.mark.gpu


def rnd(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def build_chain(g, A, X, Y):
    a, x, y = g.input(A), g.input(X), g.input(Y)
    return g.tanh(a * x + y) * g.exp(-0.5 * x * x) + g.sqrt(abs(y) + 1e-3)


@pytest.mark.parametrize("specialize", [True, False])
def test_map_chain_fuses_into_one_kernel(dev, stream, specialize):
    rows, cols = 64, 1024
    a, x, y = rnd((rows, cols), 1), rnd((rows, cols), 2), rnd((rows, cols), 3)
    A, X, Y = dev.from_numpy(a), dev.from_numpy(x), dev.from_numpy(y)
    out = dev.empty((rows, cols), np.float32)
    g = Graph(dev, rows, cols, specialize=specialize)
    g.output(build_chain(g, A, X, Y), out)
    g.compile()
    assert g.kernel_count() == 1
    assert ("fused_map" if specialize else "map_tape") in g.describe()
    g.launch(stream)
    stream.check()
    want = oracle.fused_map(a.ravel(), x.ravel(), y.ravel())
    bound = oracle.fused_map_bound(a.ravel(), x.ravel(), y.ravel(), 2.0) + 0.5 * np.spacing(np.abs(want))
    assert (np.abs(out.download().ravel().astype(np.float64) - want) <= bound).all()  # 2 ulp per primitive map, propagated
    g.close()


def test_softmax_by_hand_plans_map_reduce_map(dev, stream):
    rows, cols = 33, 512
    m = (2 * rnd((rows, cols), 4)).astype(np.float32)
    M = dev.from_numpy(m)
    out = dev.empty((rows, cols), np.float32)
    g = Graph(dev, rows, cols)
    x = g.input(M)
    e = g.exp(x - g.row_max(x))
    g.output(e / g.row_sum(e), out)
    g.compile()
    plan = g.describe()
    assert plan.count("map_tape") == 2 and "row_max" in plan and "row_sum" in plan and g.kernel_count() == 4
    g.launch(stream)
    stream.check()
    assert np.allclose(out.download(), oracle.row_softmax(m), rtol=1e-5, atol=1e-38)
    # the built-in softmax node gives the same answer in one kernel
    out2 = dev.empty((rows, cols), np.float32)
    g2 = Graph(dev, rows, cols)
    g2.output(g2.softmax(g2.input(M)), out2)
    g2.compile()
    assert g2.kernel_count() == 1
    g2.launch(stream)
    stream.check()
    assert np.allclose(out2.download(), oracle.row_softmax(m), rtol=1e-5, atol=1e-38)


def mse_graph(dev, rows, cols, specialize, want=("W", "x", "b", "loss"), seed=3001):
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    W, x, b, t = f(rows, cols), f(rows, cols), f(cols), f(rows, cols)
    bufs = {k: dev.from_numpy(v) for k, v in dict(W=W, x=x, b=b, t=t).items()}
    g = Graph(dev, rows, cols, specialize=specialize)
    nW, nx, nt = g.input(bufs["W"]), g.input(bufs["x"]), g.input(bufs["t"])
    nb = g.input(bufs["b"], L.SHAPE_ROWVEC)
    loss = g.mean(g.square(g.tanh(nW * nx + nb) - nt))
    gW, gx, gb = g.grad(loss, [nW, nx, nb])
    outs = {}
    for name, node, shape in (("W", gW, (rows, cols)), ("x", gx, (rows, cols)), ("b", gb, (cols,)), ("loss", loss, (1,))):
        if name in want:
            outs[name] = dev.empty(shape, np.float32)
            g.output(node, outs[name])
    g.compile()
    return g, (W, x, b, t), outs


def normwise(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())


@pytest.mark.parametrize("specialize", [True, False])
@pytest.mark.parametrize("rows,cols", [(40, 512), (17, 36)])
def test_autodiff_of_tanh_mse(dev, stream, specialize, rows, cols):
    g, (W, x, b, t), outs = mse_graph(dev, rows, cols, specialize)
    plan = g.describe()
    if specialize:
        assert g.kernel_count() == 1 and "mse_tanh_bwd" in plan
    else:
        assert "mse_tanh" not in plan and "map_tape" in plan and "col_sum" in plan
    g.launch(stream)
    stream.check()
    rW, rx, rb = oracle.mse_tanh_bwd(W, x, b, t)
    # the generic path differentiates 1 - tanh^2 from a rounded tanh: same tolerance norm-wise
    assert normwise(outs["W"].download(), rW) <= 1e-5
    assert normwise(outs["x"].download(), rx) <= 1e-5
    assert normwise(outs["b"].download(), rb) <= 1e-5
    assert outs["loss"].download()[0] == pytest.approx(oracle.mse_tanh_fwd(W, x, b, t), rel=1e-5)
    g.close()


def test_generic_backward_shares_one_kernel_for_dW_and_dx(dev, stream):
    g, _, _ = mse_graph(dev, 24, 128, specialize=False, want=("W", "x"))
    plan = g.describe()
    assert g.kernel_count() == 1 and "outputs=2" in plan
    g.close()


def test_partial_outputs_still_select_the_fused_kernel(dev, stream):
    g, (W, x, b, t), outs = mse_graph(dev, 24, 128, specialize=True, want=("b",))
    assert "mse_tanh_bwd" in g.describe()
    g.launch(stream)
    stream.check()
    assert normwise(outs["b"].download(), oracle.mse_tanh_bwd(W, x, b, t)[2]) <= 1e-5
    g2, (W, x, b, t), outs = mse_graph(dev, 24, 128, specialize=True, want=("loss",))
    assert "mse_tanh_fwd" in g2.describe()
    g2.launch(stream)
    stream.check()
    assert outs["loss"].download()[0] == pytest.approx(oracle.mse_tanh_fwd(W, x, b, t), rel=1e-5)


def test_gradients_of_assorted_ops_against_float64(dev, stream):
    """loss = sum( softmax(x*s) * log(1 + exp(y)) ) + mean( sqrt(x*x + 1) / (2 + cos(y)) ) with s a row
    vector; gradients by the graph vs central differences of a float64 numpy evaluation."""
    rows, cols = 6, 16
    x, y, s = rnd((rows, cols), 21), rnd((rows, cols), 22), (1 + 0.3 * rnd(cols, 23)).astype(np.float32)
    X, Y, S = dev.from_numpy(x), dev.from_numpy(y), dev.from_numpy(s)
    g = Graph(dev, rows, cols)
    nx, ny, ns = g.input(X), g.input(Y), g.input(S, L.SHAPE_ROWVEC)
    sp = g.log(1.0 + g.exp(ny))
    loss = g.sum(g.softmax(nx * ns) * sp) + g.mean(g.sqrt(nx * nx + 1.0) / (2.0 + g.unary("cos", ny)))
    gx, gy, gs = g.grad(loss, [nx, ny, ns])
    ox, oy, os_, ol = dev.empty((rows, cols), np.float32), dev.empty((rows, cols), np.float32), dev.empty(cols, np.float32), dev.empty(1, np.float32)
    for n, o in ((gx, ox), (gy, oy), (gs, os_), (loss, ol)):
        g.output(n, o)
    g.compile()
    g.launch(stream)
    stream.check()

    def f(xv, yv, sv):
        z = xv * sv[None, :]
        e = np.exp(z - z.max(axis=1, keepdims=True))
        sm = e / e.sum(axis=1, keepdims=True)
        return (sm * np.log1p(np.exp(yv))).sum() + (np.sqrt(xv * xv + 1) / (2 + np.cos(yv))).mean()

    x64, y64, s64 = x.astype(np.float64), y.astype(np.float64), s.astype(np.float64)
    assert ol.download()[0] == pytest.approx(f(x64, y64, s64), rel=2e-6)

    def fd(arr, idx, which):
        eps = 1e-5
        p, m = arr.copy(), arr.copy()
        p[idx] += eps
        m[idx] -= eps
        args_p = {"x": (p, y64, s64), "y": (x64, p, s64), "s": (x64, y64, p)}[which]
        args_m = {"x": (m, y64, s64), "y": (x64, m, s64), "s": (x64, y64, m)}[which]
        return (f(*args_p) - f(*args_m)) / (2 * eps)

    got_x, got_y, got_s = ox.download(), oy.download(), os_.download()
    for idx in [(0, 0), (3, 7), (5, 15)]:
        assert got_x[idx] == pytest.approx(fd(x64, idx, "x"), rel=2e-4, abs=2e-6)
        assert got_y[idx] == pytest.approx(fd(y64, idx, "y"), rel=2e-4, abs=2e-6)
    for idx in [(0,), (9,)]:
        assert got_s[idx] == pytest.approx(fd(s64, idx, "s"), rel=2e-4, abs=2e-6)
    g.close()


def test_graph_errors(dev):
    A = dev.from_numpy(np.zeros((4, 8), np.float32))
    small = dev.empty(4, np.float32)
    g = Graph(dev, 4, 8)
    a = g.input(A)
    with pytest.raises(L.VrhiError) as e:
        g.grad(a, [a])  # loss must be a scalar
    assert e.value.status == L.ERR_GRAPH
    with pytest.raises(L.VrhiError) as e:
        g.compile()  # no outputs
    assert e.value.status == L.ERR_GRAPH
    g.output(a * 2.0, small)
    with pytest.raises(L.VrhiError) as e:
        g.compile()  # output buffer too small
    assert e.value.status == L.ERR_SIZE
    with pytest.raises(L.VrhiError):
        g.input(small)  # too small for a full input
    g.close()
