"""GPU: the map, row and backward operators at the full shapes of the workload description
(2^28 elements; [65536, 4096]; [32768, 4096]) against the CPU oracle.

The smaller parity tests cannot see an index-width, grid-cap or tail fault that only shows at a
gibibyte per array; these can.  Inputs are the seeded device-generated arrays the benchmark uses
(bench.baseline_inputs) and the checks are the benchmark's own (bench.check_*): windows of the map's
output including its head and tail, rows spread over the matrices including the first and the last,
and, for the backward, all of db and the loss against the oracle's sum over every row.
Tolerances: the chain inside the bound 2-ulp primitives imply; everything else 1e-5 relative.
"""
import numpy as np
import pytest

import bench
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture()
def tstream(dev):
    ts = torch.cuda.Stream(device=dev.ordinal)
    st = dev.wrap_stream(ts.cuda_stream)
    yield st
    st.check()
    st.close()


def test_fused_map_baseline_shape(dev, tstream):
    a, x, y = bench.baseline_inputs(torch, f"cuda:{dev.ordinal}", 2)
    n = a.numel()
    assert n == 1 << 28
    out = torch.zeros_like(x)
    torch.cuda.synchronize()
    A, X, Y, O = (dev.wrap_tensor(t) for t in (a, x, y, out))
    ops.fused_map(tstream, A, X, Y, O, n)
    tstream.check()
    ok, worst = bench.check_fused_map(a, x, y, out)
    assert ok, f"fused_map at 2^28: error reaches {worst:.2f} x the allowed bound"
    # the same chain as a generic tape (compiled at first use, or interpreted where no run-time compiler exists)
    tp = ops.Tape(3)
    u = tp.op("fma", tp.input(0), tp.input(1), tp.input(2))
    e = tp.op("exp", tp.op("mul", tp.op("mul", tp.const(-0.5), tp.input(1)), tp.input(1)))
    q = tp.op("sqrt", tp.op("add", tp.op("abs", tp.input(2)), tp.const(1e-3)))
    tp.output(tp.op("fma", tp.op("tanh", u), e, q))
    out.zero_()
    torch.cuda.synchronize()
    ops.map_tape(tstream, tp, [A, X, Y], [O], n // 4096, 4096)
    tstream.check()
    ok, worst = bench.check_fused_map(a, x, y, out)
    assert ok, f"map_tape at 2^28: error reaches {worst:.2f} x the allowed bound"
    assert bool((out != 0).any().item())


def test_row_ops_baseline_shape(dev, tstream):
    (m,) = bench.baseline_inputs(torch, f"cuda:{dev.ordinal}", 3)
    R, Cc = m.shape
    assert (R, Cc) == (65536, 4096)
    device = m.device
    sm = torch.zeros_like(m)
    rs, rm = torch.zeros(R, device=device), torch.zeros(R, device=device)
    torch.cuda.synchronize()
    M, SM, RS, RM = (dev.wrap_tensor(t) for t in (m, sm, rs, rm))
    ops.row_sum(tstream, M, RS, R, Cc)
    ops.row_max(tstream, M, RM, R, Cc)
    ops.row_softmax(tstream, M, SM, R, Cc)
    tstream.check()
    ok, worst = bench.check_rows(m, rs, rm, sm)
    assert ok, f"row ops at [65536,4096]: {worst:.2f} x tolerance"
    # every row of the softmax sums to one, every row maximum is attained in its row: whole-matrix properties
    assert float((sm.sum(dim=1, dtype=torch.float64) - 1.0).abs().max().item()) <= 1e-5
    assert bool((m.max(dim=1).values == rm).all().item())
    first = sm.clone()
    sm.zero_(); rs.zero_(); rm.zero_()
    torch.cuda.synchronize()
    ops.row_stats_softmax(tstream, M, RS, RM, SM, R, Cc)
    tstream.check()
    ok, worst = bench.check_rows(m, rs, rm, sm)
    assert ok, f"row_stats_softmax at [65536,4096]: {worst:.2f} x tolerance"
    assert bool(torch.equal(first, sm))   # the one-pass kernel and the softmax kernel give the same bits


def test_backward_baseline_shape(dev, tstream):
    W, x, b, t = bench.baseline_inputs(torch, f"cuda:{dev.ordinal}", 4)
    R, Cc = W.shape
    assert (R, Cc) == (32768, 4096)
    device = W.device
    dW, dx = torch.zeros_like(W), torch.zeros_like(W)
    db, loss = torch.zeros(Cc, device=device), torch.zeros(4, device=device)
    torch.cuda.synchronize()
    bufs = [dev.wrap_tensor(v) for v in (W, x, b, t, dW, dx, db, loss)]
    ops.mse_tanh_bwd(tstream, *bufs[:7], R, Cc, 0.0, bufs[7])
    tstream.check()
    denom = float(R * Cc)
    ok, worst = bench.check_mse(W, x, b, t, denom, dW, dx, 0, db=db, loss=loss[0].item())
    assert ok, f"mse_tanh_bwd at [32768,4096]: {worst:.2f} x tolerance"
    # two row shards with the whole problem's denominator: db and the loss add up to the whole (the form N > 1 ranks use)
    half = R // 2
    parts = []
    for lo in (0, half):
        pdb, pl = torch.zeros(Cc, device=device), torch.zeros(4, device=device)
        sW, sx, st_ = W[lo:lo + half], x[lo:lo + half], t[lo:lo + half]
        sdW, sdx = dW[lo:lo + half], dx[lo:lo + half]
        torch.cuda.synchronize()
        sb = [dev.wrap_tensor(v) for v in (sW, sx, b, st_, sdW, sdx, pdb, pl)]
        ops.mse_tanh_bwd(tstream, *sb[:7], half, Cc, denom, sb[7])
        tstream.check()
        parts.append((pdb, pl))
    ok, worst = bench.check_mse(W, x, b, t, denom, dW, dx, 0, db=parts[0][0] + parts[1][0], loss=(parts[0][1][0] + parts[1][1][0]).item())
    assert ok, f"row shards of mse_tanh_bwd at [32768,4096]: {worst:.2f} x tolerance"
    lf = torch.zeros(4, device=device)
    torch.cuda.synchronize()
    ops.mse_tanh_fwd(tstream, *bufs[:4], dev.wrap_tensor(lf), R, Cc)
    tstream.check()
    ok, worst = bench.check_mse(W, x, b, t, denom, loss=lf[0].item())
    assert ok, f"mse_tanh_fwd at [32768,4096]: {worst:.2f} x tolerance"
