"""GPU: fused map chain and the generic tape kernel against the binary64 CPU oracle."""
import numpy as np
import pytest

import oracle
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu

# Tolerance of the fused chain.  "Maps within 2 ulp" is a statement about each primitive map
# (checked one by one in test_tape_primitives_within_2_ulp).  For the composite
# tanh(a*x+y)*exp(-x*x/2) + sqrt(|y|+1e-3) an ulp of the result is not a usable unit, because the
# two terms can cancel; what 2-ulp primitives imply for the result is the first-order forward
# error bound  2 * sum_t |d out/d t| * ulp(t)  over the chain's intermediates t, which the oracle
# evaluates in binary64 (oracle.fused_map_bound).  The kernel must stay inside that bound on every
# element; on top of it the error measured in ulps of the largest intermediate is held below
# CHAIN_SCALED_ULPS, which is tighter over most of the input range.
PRIMITIVE_ULPS = 2.0
CHAIN_SCALED_ULPS = 4.0


def chain_inputs(n, seed=1001):
    rng = np.random.default_rng(seed)
    return (rng.uniform(-1, 1, n).astype(np.float32), rng.standard_normal(n).astype(np.float32),
            rng.standard_normal(n).astype(np.float32))


def check_chain(got, a, x, y):
    want, scale = oracle.fused_map(a, x, y, want_scale=True)
    bound = oracle.fused_map_bound(a, x, y, PRIMITIVE_ULPS)
    err_abs = np.abs(got.astype(np.float64) - want.astype(np.float64))
    # `want` is the binary64 value rounded once to binary32: allow that half ulp on top of the bound
    slack = 0.5 * np.spacing(np.abs(want)).astype(np.float64)
    worst = (err_abs / (bound + slack)).max()
    assert worst <= 1.0, f"error reaches {worst:.2f} x the 2-ulp-per-primitive bound"
    unit = np.spacing(np.maximum(scale, np.abs(want)).astype(np.float32)).astype(np.float64)
    scaled = err_abs / unit
    assert scaled.max() <= CHAIN_SCALED_ULPS, f"max error {scaled.max():.2f} ulp of the largest intermediate"
    return worst, scaled.max()


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1023, 4099, 1 << 20, (1 << 22) + 3])
def test_fused_map_matches_oracle(dev, stream, n):
    a, x, y = chain_inputs(n)
    A, X, Y = (dev.from_numpy(v) for v in (a, x, y))
    out = dev.empty(n, np.float32)
    ops.fused_map(stream, A, X, Y, out, n)
    stream.check()
    check_chain(out.download(), a, x, y)
    for b in (A, X, Y, out):
        b.close()


def test_fused_map_golden(dev, stream, golden):
    a, x, y = golden["map_a"], golden["map_x"], golden["map_y"]
    A, X, Y = (dev.from_numpy(v) for v in (a, x, y))
    out = dev.empty(a.size, np.float32)
    ops.fused_map(stream, A, X, Y, out, a.size)
    stream.check()
    got = out.download()
    unit = np.spacing(np.maximum(np.abs(golden["map_out"]), 1.0).astype(np.float32))
    assert (np.abs(got - golden["map_out"]) <= 4 * unit).all()


def test_fused_map_extreme_inputs(dev, stream):
    x = np.array([0.0, -0.0, 1e-30, 30.0, -30.0, 8.0, 1e-4, -1e-4] * 4, dtype=np.float32)
    a = np.linspace(-1, 1, x.size).astype(np.float32)
    y = np.array([0.0, 1e-20, -5.0, 5.0, 1e3, -1e3, 0.5, -0.5] * 4, dtype=np.float32)
    A, X, Y = (dev.from_numpy(v) for v in (a, x, y))
    out = dev.empty(x.size, np.float32)
    ops.fused_map(stream, A, X, Y, out, x.size)
    stream.check()
    got = out.download()
    assert np.isfinite(got).all()
    check_chain(got, a, x, y)


def chain_tape():
    t = ops.Tape(3)
    a, x, y = t.input(0), t.input(1), t.input(2)
    u = t.op("fma", a, x, y)
    th = t.op("tanh", u)
    e = t.op("exp", t.op("mul", t.op("mul", t.const(-0.5), x), x))
    q = t.op("sqrt", t.op("add", t.op("abs", y), t.const(1e-3)))
    t.output(t.op("fma", th, e, q))
    return t


def run_tape_both_ways(dev, stream, tape, inputs, out_shapes, rows, cols):
    """Runs the tape as a kernel compiled for it and through the interpreting kernel; the two must agree bit for
    bit.  Where the compiled path applies (columns a multiple of 4) it must really have run."""
    outs_c = [dev.empty(s, np.float32) for s in out_shapes]
    outs_i = [dev.empty(s, np.float32) for s in out_shapes]
    before = ops.tape_jit_stats()["launches"]
    ops.map_tape(stream, tape, inputs, outs_c, rows, cols)
    compiled_ran = ops.tape_jit_stats()["launches"] - before
    ops.map_tape(stream, tape, inputs, outs_i, rows, cols, interpret=True)
    assert ops.tape_jit_stats()["launches"] - before == compiled_ran      # the flag really selects the interpreter
    stream.check()
    assert compiled_ran == (1 if cols % 4 == 0 else 0)
    got_c, got_i = [o.download() for o in outs_c], [o.download() for o in outs_i]
    info = ops.tape_jit_stats()
    for c, i in zip(got_c, got_i):
        if info["compiler_version"] == info["built_version"] or not compiled_ran:
            assert np.array_equal(c.view(np.uint32), i.view(np.uint32)), "compiled and interpreted tape differ"
        else:   # another compiler version: its math library may round the last place differently
            assert np.allclose(c, i, rtol=3e-7, atol=1e-37, equal_nan=True)
    return got_c


@pytest.mark.parametrize("rows,cols", [(1, 4096), (64, 1024), (7, 36), (5, 13), (1, 1), (3, 4), (1000, 1028), (1, (1 << 20) + 4)])
def test_tape_runs_the_same_chain(dev, stream, rows, cols):
    n = rows * cols
    a, x, y = chain_inputs(n, seed=7)
    A, X, Y = (dev.from_numpy(v) for v in (a, x, y))
    got, = run_tape_both_ways(dev, stream, chain_tape(), [A, X, Y], [n], rows, cols)
    check_chain(got, a, x, y)


UNARY_RANGES = {"tanh": (-12, 12), "exp": (-80, 80), "sqrt": (0, 1e6), "abs": (-5, 5), "neg": (-5, 5), "square": (-1e3, 1e3),
                "recip": (0.01, 100), "log": (1e-6, 1e6), "sigmoid": (-30, 30), "relu": (-5, 5), "cos": (-20, 20),
                "sin": (-20, 20), "rsqrt": (1e-4, 1e4)}


@pytest.mark.parametrize("op", sorted(UNARY_RANGES))
def test_tape_primitives_within_2_ulp(dev, stream, op):
    lo, hi = UNARY_RANGES[op]
    rng = np.random.default_rng(11)
    x = rng.uniform(lo, hi, 1 << 16).astype(np.float32)
    if op in ("tanh", "sigmoid", "exp"):
        x[:4096] = rng.uniform(-1e-3, 1e-3, 4096).astype(np.float32)  # near zero, where relative accuracy is hardest
    X = dev.from_numpy(x)
    t = ops.Tape(1)
    t.output(t.op(op, t.input(0)))
    got, = run_tape_both_ways(dev, stream, t, [X], [x.size], 1, x.size)
    want = oracle.unary(op, x)
    ok = np.isfinite(want) & (np.abs(want) > 1e-37)
    # cos/sin: error measured against the function's scale near its zeros, as libm accuracy tables do
    err = oracle.ulp_diff(got[ok], want[ok]) if op not in ("cos", "sin") else \
        np.abs(got[ok].astype(np.float64) - want[ok]) / np.spacing(np.maximum(np.abs(want[ok]), np.float32(0.25)))
    assert err.max() <= 2.0, f"{op}: {err.max():.2f} ulp"


def test_tape_broadcasts_and_multiple_outputs(dev, stream):
    rows, cols = 37, 256
    rng = np.random.default_rng(3)
    m = rng.standard_normal((rows, cols)).astype(np.float32)
    rv = rng.standard_normal(cols).astype(np.float32)
    cv = rng.standard_normal(rows).astype(np.float32)
    sc = np.array([1.75], dtype=np.float32)
    for cols_used in (cols, 255):  # vector path and scalar path
        mm = np.ascontiguousarray(m[:, :cols_used])
        rr = np.ascontiguousarray(rv[:cols_used])
        M, RV, CV, SC = dev.from_numpy(mm), dev.from_numpy(rr), dev.from_numpy(cv), dev.from_numpy(sc)
        t = ops.Tape(4, row_vectors=[1], col_vectors=[2], scalars=[3])
        s = t.op("add", t.op("mul", t.input(0), t.input(1)), t.input(2))
        t.output(s)
        t.output(t.op("mul", t.op("max", s, t.const(0.0)), t.input(3)))
        o1, o2 = run_tape_both_ways(dev, stream, t, [M, RV, CV, SC], [mm.shape, mm.shape], rows, cols_used)
        want1 = (mm * rr[None, :]).astype(np.float32) + cv[:, None]
        assert np.array_equal(o1, want1)
        assert np.array_equal(o2, np.maximum(want1, 0) * sc[0])


def test_tape_errors(dev, stream):
    X = dev.from_numpy(np.zeros(64, np.float32))
    out = dev.empty(64, np.float32)
    t = ops.Tape(1)
    t.output(t.op("add", t.input(0), 5))  # value 5 is not defined yet
    with pytest.raises(L.VrhiError) as e:
        ops.map_tape(stream, t, [X], [out], 1, 64)
    assert e.value.status == L.ERR_INVALID
    t = ops.Tape(1)
    t.output(t.op("neg", t.input(0)))
    with pytest.raises(L.VrhiError) as e:
        ops.map_tape(stream, t, [X], [out], 2, 64)  # 128 elements do not fit
    assert e.value.status == L.ERR_SIZE


def test_compiled_tape_covers_every_operation_and_is_cached(dev, stream):
    """One tape through every opcode: compiled and interpreted kernels must agree bit for bit, a second
    launch must reuse the compiled kernel, and a compiled tape can be recorded into a sequence."""
    rows, cols = 33, 512
    rng = np.random.default_rng(21)
    a = rng.uniform(0.1, 3.0, (rows, cols)).astype(np.float32)
    b = rng.uniform(-2.0, 2.0, (rows, cols)).astype(np.float32)
    A, B = dev.from_numpy(a), dev.from_numpy(b)
    t = ops.Tape(2)
    x, y = t.input(0), t.input(1)
    acc = t.op("add", x, y)
    for name in ("sub", "mul", "div", "max", "min", "eq"):
        acc = t.op("add", acc, t.op(name, x, y))
    for name in ("neg", "abs", "square", "relu", "sign", "step", "sqrt", "rsqrt", "recip", "exp", "log", "tanh", "sigmoid", "cos", "sin"):
        acc = t.op("add", acc, t.op(name, x))
    acc = t.op("fma", acc, t.const(0.5), y)
    t.output(acc)
    t.output(t.op("sigmoid", y))
    before = ops.tape_jit_stats()
    o1, o2 = run_tape_both_ways(dev, stream, t, [A, B], [(rows, cols), (rows, cols)], rows, cols)
    mid = ops.tape_jit_stats()
    assert mid["compiled"] - before["compiled"] == 1
    assert np.all(np.isfinite(o1)) and np.all((o2 > 0) & (o2 < 1))
    again = [dev.empty((rows, cols), np.float32) for _ in range(2)]
    ops.map_tape(stream, t, [A, B], again, rows, cols)
    assert ops.tape_jit_stats()["compiled"] == mid["compiled"]          # cached
    with stream.record() as seq:                                       # compiled before: recordable
        ops.map_tape(stream, t, [A, B], again, rows, cols)
    for o in again:
        o.fill(0, stream=stream)
    seq.launch()
    stream.check()
    assert np.array_equal(again[0].download(), o1) and np.array_equal(again[1].download(), o2)
    seq.close()


def test_tape_output_summed_over_columns_inside_the_kernel(dev, stream):
    """An output flagged col_sum is never stored in full: the compiled kernel adds it up column by column
    (fixed order: the same bits on every run) and a [cols] vector comes out."""
    rows, cols = 301, 1024
    rng = np.random.default_rng(8)
    w = rng.standard_normal((rows, cols)).astype(np.float32)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    b = rng.standard_normal(cols).astype(np.float32)
    W, X, B = dev.from_numpy(w), dev.from_numpy(x), dev.from_numpy(b)
    t = ops.Tape(3, row_vectors=[2])
    u = t.op("tanh", t.op("fma", t.input(0), t.input(1), t.input(2)))
    t.output(u)
    t.output(t.op("mul", u, t.input(0)), col_sum=True)
    full, sums = dev.empty((rows, cols), np.float32), dev.empty((cols,), np.float32)
    ops.map_tape(stream, t, [W, X, B], [full, sums], rows, cols)
    stream.check()
    want_u = np.tanh(w.astype(np.float64) * x + b[None, :])
    got_u, got_s = full.download(), sums.download()
    assert np.abs(got_u - want_u).max() < 1e-6
    want_s = (want_u * w).sum(axis=0)
    assert np.abs(got_s - want_s).max() <= 1e-5 * np.abs(want_u * w).sum(axis=0).max()
    again = dev.empty((cols,), np.float32)
    ops.map_tape(stream, t, [W, X, B], [full, again], rows, cols)
    stream.check()
    assert np.array_equal(again.download().view(np.uint32), got_s.view(np.uint32))     # deterministic
    with pytest.raises(L.VrhiError) as e:                                               # the interpreter has no such epilogue
        ops.map_tape(stream, t, [W, X, B], [full, again], rows, cols, interpret=True)
    assert e.value.status == L.ERR_UNSUPPORTED
