"""Benchmark of the data-parallel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workloads all|main]

Headline workload (one "step" = one whole image): the Julia-set escape-time map on a
16384 x 16384 binary32 grid over [-1.6, 1.6]^2, c = -0.8 + 0.156i, max_iter = 4096, uint32
counts, exact (uncontracted) arithmetic.  With N > 1 the rows are dealt to the ranks in cyclic
128-row chunks and the image is all-gathered (NCCL) at the end of every step, as the workload
states; the compute-only figure is reported beside it.  Metric: Gpixel-iters/s = (sum over
pixels of the iteration count) / time; the count total is an exact property of the workload
(7 055 521 946, from the CPU oracle, stored in tests/golden/golden.npz).

The JSON line also carries: `roofline` (FP32 issue-rate bound for the escape-time kernel: 8
binary32 operations per pixel-iteration against an FFMA-chain probe measured in the same run),
`cpu_baseline` (the CPU oracle on the box's host cores), `e2e` (through the public API with the
result landing in pinned host memory), `other_workloads` (1080p Mandelbrot frames, the fused map
chain, row reductions / softmax, tanh-MSE forward and backward: achieved HBM GB/s against the
measured copy bandwidth) and `clocks`.

`--impl reference` times the CPU restatement of the path (the reference project ships no
runnable implementation of it) on all host threads, on a bounded row sample of the same image.
"""
from __future__ import annotations

import argparse
import json
import copy
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

JULIA = dict(W=16384, H=16384, x0=-1.6, x1=1.6, y0=-1.6, y1=1.6, cr=-0.8, ci=0.156, max_iter=4096)
WORKLOAD_NAME = "julia 16384x16384 [-1.6,1.6]^2 c=-0.8+0.156i max_iter=4096 u32 exact"
OPS_PER_ITER = 8  # a=zr*zr b=zi*zi s=a+b t=zr*zi t+t (..)+ci a-b (..)+cr


def golden_total() -> int:
    g = np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))
    return int(g["julia_16k_digest"][0])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for line in open(self.path):
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def run_reference(args):
    """CPU arm: the oracle on all host threads, on a bounded row sample of the Julia image."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    J = JULIA
    dx, dy = oracle.grid_steps(J["x0"], J["x1"], J["y0"], J["y1"], J["W"], J["H"])
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use the whole host
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = oracle.num_threads()

    def sample(stride):
        t = time.perf_counter()
        _, total = oracle.escape_time(oracle.JULIA, J["W"], J["H"], J["x0"], J["y0"], dx, dy, J["cr"], J["ci"], J["max_iter"],
                                      row_begin=stride // 2 if stride > 1 else 0, row_step=stride, want_image=False)
        return total, time.perf_counter() - t

    _, probe_s = sample(64)
    stride = 1
    while probe_s * 64 / stride > 6.0 and stride < 64:  # keep one step under ~6 s
        stride *= 2
    for _ in range(args.warmup):
        sample(stride)
    iters, secs = 0, 0.0
    for _ in range(args.steps):
        n, s = sample(stride)
        iters += n
        secs += s
    value = iters / secs / 1e9
    desc = f"every {stride}th row of the image ({J['H'] // stride} rows x {J['W']} px per step)" if stride > 1 else "the whole image per step"
    line = {"impl": "reference", "metric": "Gpixel-iters/s", "value": value, "unit": "Gpixel-iters/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "sample": desc},
            "cpu_baseline": {"value": value, "unit": "Gpixel-iters/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": "Gpixel-iters/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference project has no runnable implementation of this path; this is the CPU restatement (oracle/) on all host threads"}
    print(json.dumps(line), flush=True)


def time_launches(dev, st, fn, iters, warmup=3):
    """Average milliseconds per call of fn(), CUDA events on the launching stream."""
    for _ in range(warmup):
        fn()
    e0, e1 = dev.event(), dev.event()
    st.synchronize()
    e0.record(st)
    for _ in range(iters):
        fn()
    e1.record(st)
    e1.synchronize()
    ms = e0.elapsed_ms(e1) / iters
    e0.close(); e1.close()
    return ms


# ------------------------------------------------------------------------------------------------
# Checks of the HBM-bound workloads at their full shapes.  Test infrastructure: the CPU oracle is
# the checker here, outside every timed region; tests/test_baseline_shapes_gpu.py runs the same
# functions.  Tolerances: the fused chain inside the bound that 2-ulp primitives imply (and within
# 4 ulp of its largest intermediate); reductions, softmax, loss and gradients within 1e-5 relative
# (sums against the sum of magnitudes, gradients norm-wise).
RTOL = 1e-5


def spread(n, k):
    """k indices spread over range(n), first and last included."""
    return np.unique(np.linspace(0, n - 1, min(k, n)).astype(np.int64))


def baseline_inputs(torch, device, config):
    """Seeded inputs of one workload at its full shape, generated on the device."""
    gen = torch.Generator(device=device)

    def randn(shape, seed, scale=1.0):
        gen.manual_seed(seed)
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        return t * scale if scale != 1.0 else t

    if config == 2:      # fused map chain: x, y ~ N(0,1), a ~ U(-1,1), 2^28 elements
        n = 1 << 28
        gen.manual_seed(1003)
        a = torch.rand(n, generator=gen, device=device, dtype=torch.float32) * 2 - 1
        return a, randn(n, 1001), randn(n, 1002)
    if config == 3:      # [65536, 4096], N(0, 4) read as sigma = 2
        return (randn((65536, 4096), 2001, 2.0),)
    if config == 4:      # W, x, t [32768, 4096], b [4096], N(0,1)
        return randn((32768, 4096), 3001), randn((32768, 4096), 3002), randn(4096, 3004), randn((32768, 4096), 3003)
    raise ValueError(config)


def check_fused_map(a, x, y, out):
    """Windows of the chain's output (head, tail and 62 windows between) against the binary64 oracle.
    -> (ok, worst error as a fraction of the allowed bound)."""
    import oracle

    n = out.numel()
    win = 4096
    starts = sorted(set([0, max(0, n - 65536)] + [int(v) // 16 * 16 for v in np.linspace(0, max(0, n - win), 62)]))
    worst = 0.0
    for s0 in starts:
        s1 = min(n, s0 + (65536 if s0 in (0, max(0, n - 65536)) else win))
        ha, hx, hy, ho = (t[s0:s1].cpu().numpy() for t in (a, x, y, out))
        want, scale = oracle.fused_map(ha, hx, hy, want_scale=True)
        bound = oracle.fused_map_bound(ha, hx, hy, 2.0) + 0.5 * np.spacing(np.abs(want)).astype(np.float64)
        err = np.abs(ho.astype(np.float64) - want.astype(np.float64))
        unit = np.spacing(np.maximum(scale, np.abs(want)).astype(np.float32)).astype(np.float64)
        worst = max(worst, float((err / bound).max()), float((err / unit).max()) / 4.0)
    return worst <= 1.0, worst


def check_rows(m, row_sum=None, row_max=None, softmax=None, k=64):
    """k rows spread over the matrix (first and last included) against the oracle.
    -> (ok, worst error as a fraction of the tolerance)."""
    import oracle

    import torch

    rows = spread(m.shape[0], k)
    idx = torch.from_numpy(rows).to(m.device)
    hm = m[idx].cpu().numpy()
    worst = 0.0
    if row_sum is not None:
        scale = np.abs(hm).astype(np.float64).sum(axis=1)
        worst = max(worst, float((np.abs(row_sum[idx].cpu().numpy() - oracle.row_sum(hm)) / (RTOL * scale + 1e-30)).max()))
    if row_max is not None and not np.array_equal(row_max[idx].cpu().numpy(), oracle.row_max(hm)):
        worst = float("inf")
    if softmax is not None:
        got, want = softmax[idx].cpu().numpy().astype(np.float64), oracle.row_softmax(hm).astype(np.float64)
        worst = max(worst, float((np.abs(got - want) / (RTOL * np.abs(want) + 1e-38)).max()),
                    float(np.abs(got.sum(axis=1) - 1.0).max() / 1e-5))
    return worst <= 1.0, worst


def check_mse(W, x, b, t, denom, dW=None, dx=None, row0=0, db=None, loss=None, k=256):
    """Gradients and loss of the tanh-MSE problem.  W, x, t are the WHOLE problem (the oracle sums db
    and the loss over all rows); dW / dx may be a row shard starting at row0, checked on k rows
    spread over the shard; db and loss, when given, are the whole problem's.
    -> (ok, worst norm-wise error as a fraction of the tolerance)."""
    import oracle

    import torch

    worst = 0.0
    hb = b.cpu().numpy()
    if db is not None or loss is not None:
        hW, hx, ht = W.cpu().numpy(), x.cpu().numpy(), t.cpu().numpy()
        if db is not None:
            _, _, rb = oracle.mse_tanh_bwd(hW, hx, hb, ht, denom)
            worst = max(worst, float(np.abs(db.cpu().numpy().astype(np.float64) - rb).max() / np.abs(rb).max()) / RTOL)
        if loss is not None:
            want = oracle.mse_tanh_fwd(hW, hx, hb, ht, denom)
            worst = max(worst, abs(float(loss) - want) / abs(want) / RTOL)
        del hW, hx, ht
    if dW is not None:
        rows = spread(dW.shape[0], k)
        gi = torch.from_numpy(rows + row0).to(W.device)
        li = torch.from_numpy(rows).to(W.device)
        rW, rx, _ = oracle.mse_tanh_bwd(W[gi].cpu().numpy(), x[gi].cpu().numpy(), hb, t[gi].cpu().numpy(), denom)
        for got, want in ((dW[li], rW), (dx[li], rx)):
            worst = max(worst, float(np.abs(got.cpu().numpy().astype(np.float64) - want).max() / np.abs(want).max()) / RTOL)
    return worst <= 1.0, worst


def hbm_workloads(dev, st, torch, rank, world, hbm_peak, peak_kind, grp=None, graphs=True):
    """The map, row and backward workloads at their full shapes, split along the leading axis over
    `world` ranks (no collective, except the all-reduce of db and the loss), each checked against the
    oracle after its timed loop.  `grp` is the ranks' vernondsl_b200.group.Group (its all-reduce sums db and the loss).  Inputs are generated on the device (seeded).  Times are CUDA events
    on the launching stream, the maximum over ranks; GB/s is the whole job's."""
    import torch.distributed as dist

    from vernondsl_b200 import _lib as L
    from vernondsl_b200 import ops, partition

    import oracle   # the checker, outside every timed region

    oracle.set_num_threads(max(1, (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)) // world))
    out = []
    device = f"cuda:{dev.ordinal}"

    def timed(fn, iters=10):
        if world > 1:
            dist.barrier()
        ms = time_launches(dev, st, fn, iters)
        if world > 1:
            v = torch.tensor([ms], device=device)
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            ms = float(v.item())
        return ms

    def agree(ok, worst):
        if world > 1:
            v = torch.tensor([0.0 if ok else 1.0, min(worst, 1e30)], device=device, dtype=torch.float64)
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            return bool(v[0].item() == 0.0), float(v[1].item())
        return bool(ok), float(worst)

    def line(name, kernel, ms, algo_bytes, check, **extra):
        ok, worst = agree(*check)
        gbs = algo_bytes / (ms * 1e-3) / 1e9
        out.append(dict({"workload": name, "kernel": kernel, "ms": ms, "algorithmic_bytes": algo_bytes, "achieved_gbs": gbs,
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak * world, "unit": "GB/s", "frac": gbs / (hbm_peak * world),
                                      "peak_kind": peak_kind, "frac_of_nominal_8tbs": gbs / (8000.0 * world)},
                         "verified": ok, "max_err": worst}, **extra))

    # ---- fused map chain, 2^28 elements
    a, x, y = baseline_inputs(torch, device, 2)
    n = a.numel()
    o = torch.zeros_like(x)
    torch.cuda.synchronize()   # the inputs were made on torch's default stream; the kernels run on `st`
    lo, cnt = partition.leading_slice(n, world, rank)
    sa, sx, sy, so = (t[lo:lo + cnt] for t in (a, x, y, o))
    A, X, Y, O = (dev.wrap_tensor(t) for t in (sa, sx, sy, so))
    ms = timed(lambda: ops.fused_map(st, A, X, Y, O, cnt))
    st.check()
    line("fused map chain 2^28", "fused_map", ms, 16 * n, check_fused_map(sa, sx, sy, so))
    if cnt % 4096 == 0:
        # the same chain through the generic fused-tape kernel (what an arbitrary DSL chain runs on)
        tp = ops.Tape(3)
        u = tp.op("fma", tp.input(0), tp.input(1), tp.input(2))
        e = tp.op("exp", tp.op("mul", tp.op("mul", tp.const(-0.5), tp.input(1)), tp.input(1)))
        q = tp.op("sqrt", tp.op("add", tp.op("abs", tp.input(2)), tp.const(1e-3)))
        tp.output(tp.op("fma", tp.op("tanh", u), e, q))
        so.zero_(); torch.cuda.synchronize()
        before = ops.tape_jit_stats()["launches"]
        ms = timed(lambda: ops.map_tape(st, tp, [A, X, Y], [O], cnt // 4096, 4096))
        st.check()
        compiled = ops.tape_jit_stats()["launches"] > before
        line("the chain as a generic tape 2^28", "map_tape (compiled at first use)" if compiled else "map_tape (interpreted: no run-time compiler)",
             ms, 16 * n, check_fused_map(sa, sx, sy, so))
        if compiled and world == 1:
            so.zero_(); torch.cuda.synchronize()
            ms = timed(lambda: ops.map_tape(st, tp, [A, X, Y], [O], cnt // 4096, 4096, interpret=True))
            st.check()
            line("the tape interpreted 2^28", "map_tape (interpreted)", ms, 16 * n, check_fused_map(sa, sx, sy, so), bound_by="instruction issue")
    del a, x, y, o, sa, sx, sy, so
    torch.cuda.empty_cache()

    # ---- row reductions and softmax, [65536, 4096]
    (m,) = baseline_inputs(torch, device, 3)
    R, Cc = m.shape
    lo, cnt = partition.leading_slice(R, world, rank)
    sm_in = m[lo:lo + cnt]
    sm = torch.zeros_like(sm_in)
    rs, rm = torch.zeros(cnt, device=device), torch.zeros(cnt, device=device)
    torch.cuda.synchronize()
    M, SM, RS, RM = (dev.wrap_tensor(t) for t in (sm_in, sm, rs, rm))
    ms = timed(lambda: ops.row_sum(st, M, RS, cnt, Cc))
    st.check()
    line("row sum [65536,4096]", "row_sum", ms, 4 * R * Cc + 4 * R, check_rows(sm_in, row_sum=rs))
    ms = timed(lambda: ops.row_max(st, M, RM, cnt, Cc))
    st.check()
    line("row max [65536,4096]", "row_max", ms, 4 * R * Cc + 4 * R, check_rows(sm_in, row_max=rm))
    ms = timed(lambda: ops.row_softmax(st, M, SM, cnt, Cc))
    st.check()
    line("row softmax [65536,4096]", "row_softmax", ms, 8 * R * Cc, check_rows(sm_in, softmax=sm))
    sm.zero_(); rs.zero_(); rm.zero_(); torch.cuda.synchronize()
    ms = timed(lambda: ops.row_stats_softmax(st, M, RS, RM, SM, cnt, Cc))
    st.check()
    line("row sum+max+softmax one pass [65536,4096]", "row_stats_softmax", ms, 8 * R * Cc + 8 * R, check_rows(sm_in, rs, rm, sm))
    del m, sm, sm_in
    torch.cuda.empty_cache()

    # ---- tanh-MSE loss and backward, [32768, 4096]; rows split, db and the loss all-reduced
    Wt, xt, bt, tt = baseline_inputs(torch, device, 4)
    R, Cc = Wt.shape
    denom = float(R * Cc)
    lo, cnt = partition.leading_slice(R, world, rank)
    sW, sx, stt = (t[lo:lo + cnt] for t in (Wt, xt, tt))
    dWt, dxt = torch.zeros_like(sW), torch.zeros_like(sW)
    small = torch.zeros(Cc + 4, device=device)       # db [4096] and the loss in one array: one all-reduce
    dbt, lt = small[:Cc], small[Cc:Cc + 1]
    torch.cuda.synchronize()
    bW, bx, bb, bt_, bdW, bdx, bdb, bl = (dev.wrap_tensor(t) for t in (sW, sx, bt, stt, dWt, dxt, dbt, lt))
    bsmall = dev.wrap_tensor(small)

    tstream = None
    if world > 1 and grp is None:   # no peer mapping on this box: the process group's all-reduce on the same stream
        tstream = torch.cuda.ExternalStream(st.cuda_stream, device=device)

    def reduce_small():
        if world > 1 and grp is not None:
            grp.all_reduce_sum(bsmall, Cc + 1, st)   # db and the loss: one call of the library's own all-reduce
        elif world > 1:
            with torch.cuda.stream(tstream):
                dist.all_reduce(small)

    def fwd():
        ops.mse_tanh_fwd(st, bW, bx, bb, bt_, bl, cnt, Cc, denom)
        reduce_small()

    ms = timed(fwd)
    st.check()
    small.zero_(); torch.cuda.synchronize(); fwd(); st.check()
    line("tanh-MSE loss [32768,4096]", "mse_tanh_fwd" + (" + vrhi all-reduce" if world > 1 and grp is not None else " + all-reduce" if world > 1 else ""), ms, 12 * R * Cc,
         check_mse(Wt, xt, bt, tt, denom, loss=lt.item()) if rank == 0 else (True, 0.0))

    def bwd(reduce=True):
        ops.mse_tanh_bwd(st, bW, bx, bb, bt_, bdW, bdx, bdb, cnt, Cc, denom, bl)
        if reduce:
            reduce_small()

    ms = timed(bwd)
    extra = {}
    if world > 1:
        extra["ms_without_all_reduce"] = timed(lambda: bwd(False))
    st.check()
    small.zero_(); torch.cuda.synchronize(); bwd(); st.check()
    ok_rows = check_mse(Wt, xt, bt, tt, denom, dWt, dxt, lo)
    ok_sum = check_mse(Wt, xt, bt, tt, denom, db=dbt, loss=lt.item()) if rank == 0 else (True, 0.0)
    line("tanh-MSE backward dW,dx,db,loss [32768,4096]", "mse_tanh_bwd" + (" + vrhi all-reduce of db and loss" if world > 1 and grp is not None else " + all-reduce of db and loss" if world > 1 else ""), ms,
         20 * R * Cc + 8 * Cc, (ok_rows[0] and ok_sum[0], max(ok_rows[1], ok_sum[1])), **extra)
    if graphs and world == 1:
        # The same gradients through the generic path: the execution graph differentiates the loss and fuses the
        # elementwise parts into one tape, compiled at first use, whose third output (the adjoint of b) is summed over
        # the rows inside the kernel; no hand-written loss kernel is selected.
        from vernondsl_b200.graph import Graph

        dWt.zero_(); dxt.zero_(); small.zero_(); torch.cuda.synchronize()
        g = Graph(dev, R, Cc, specialize=False)
        nW, nx, nt = g.input(bW), g.input(bx), g.input(bt_)
        nb = g.input(bb, L.SHAPE_ROWVEC)
        loss = g.mean(g.square(g.tanh(nW * nx + nb) - nt))
        gW, gx, gb = g.grad(loss, [nW, nx, nb])
        g.output(gW, bdW)
        g.output(gx, bdx)
        g.output(gb, bdb)
        g.compile()
        ms = timed(lambda: g.launch(st))
        st.check()
        ok_rows = check_mse(Wt, xt, bt, tt, denom, dWt, dxt, 0)
        ok_sum = check_mse(Wt, xt, bt, tt, denom, db=dbt)
        line("the gradients from the execution graph (autodiff, no hand-written kernel)", f"graph: {g.kernel_count()} kernels", ms,
             20 * R * Cc + 8 * Cc, (ok_rows[0] and ok_sum[0], max(ok_rows[1], ok_sum[1])))
        g.close()
        small.zero_(); torch.cuda.synchronize()
        g = Graph(dev, R, Cc, specialize=False)
        nW, nx, nt = g.input(bW), g.input(bx), g.input(bt_)
        nb = g.input(bb, L.SHAPE_ROWVEC)
        g.output(g.mean(g.square(g.tanh(nW * nx + nb) - nt)), bl)
        g.compile()
        ms = timed(lambda: g.launch(st))
        st.check()
        line("the loss from the execution graph (no hand-written kernel)", f"graph: {g.kernel_count()} kernels", ms, 12 * R * Cc,
             check_mse(Wt, xt, bt, tt, denom, loss=lt.item()))
        g.close()
    return out


def frame_workloads(dev, st, torch, fp32_peak, fp32_nominal):
    """Single-GPU lines for the frame-sized escape-time workloads (launch- and drain-bound, not DRAM-sized)."""
    from vernondsl_b200 import _lib as L
    from vernondsl_b200 import ops

    out = []
    # Mandelbrot 1920x1080, max_iter 256: frames back to back on one stream, every frame checked by its exact digest
    W, H = 1920, 1080
    dx, dy = ops.grid_steps(-2.5, 1.0, -1.0, 1.0, W, H)
    img = dev.empty((H, W), np.uint32, L.IMAGE)
    p = ops.escape_params(L.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=256)
    ms = time_launches(dev, st, lambda: ops.escape_time(st, img, p), 50)
    want = [int(v) for v in np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))["mandelbrot_1080p_digest"]]
    total = want[0]

    def digest(buf):
        t = buf.as_tensor(np.uint32, (H, W)).view(-1).to(torch.int64)
        idx = torch.arange(1, H * W + 1, device=t.device, dtype=torch.int64)
        return [int(t.sum().item()), int((t * idx).sum().item()) & 0xFFFFFFFFFFFFFFFF]

    def frame_line(name, ms_frame, ok, short):
        rate = total / (ms_frame * 1e-3)
        out.append({"workload": name, "short": short, "kernel": "escape_time", "ms": ms_frame, "gpixel_iters_per_s": rate / 1e9, "verified": ok,
                    "roofline": {"bound": "fp32", "achieved": OPS_PER_ITER * rate / 1e9, "peak": fp32_peak, "unit": "Gop/s",
                                 "frac": OPS_PER_ITER * rate / 1e9 / fp32_peak, "frac_of_nominal": OPS_PER_ITER * rate / 1e9 / fp32_nominal}})

    frame_line("mandelbrot 1080p max_iter=256, 50 frames back to back on one stream", ms, digest(img) == want, "1080p, 1 stream, 1 image")
    # The same 50 launches on the same one stream into a ring of 4 images, each declared independent of the 3
    # launches before it (they write other slots): a frame's first blocks start beside the last blocks of the
    # frame before; every fourth launch is ordered behind everything before it.
    ring = [img] + [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(3)]
    p_ring = ops.escape_params(L.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=256, independent_of=3)
    turn = [0]

    def next_frame():
        ops.escape_time(st, ring[turn[0] % 4], p_ring)
        turn[0] += 1

    for b in ring:
        b.fill(0, stream=st)
    ms_ring = time_launches(dev, st, next_frame, 50)
    st.check()
    frame_line("mandelbrot 1080p ring of 4, 50 frames back to back on one stream, each launch declared independent of the 3 before it",
               ms_ring, all(digest(r) == want for r in ring), "1080p, 1 stream, ring of 4")
    # a ring of 8, each launch independent of the 7 before it: one ordered launch in eight; recorded once
    ring += [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(4)]
    p_ring8 = ops.escape_params(L.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=256, independent_of=7)
    with st.record() as seq:
        for k in range(48):
            ops.escape_time(st, ring[k % 8], p_ring8)
    for b in ring:
        b.fill(0, stream=st)
    ms_ring_seq = time_launches(dev, st, lambda: seq.launch(), 5) / 48
    st.check()
    frame_line("mandelbrot 1080p ring of 8, 48 frames recorded on one stream, each launch declared independent of the 7 before it",
               ms_ring_seq, all(digest(r) == want for r in ring), "1080p, 1 stream, ring of 8, recorded")
    seq.close()
    for b in ring[1:]:
        b.close()
    # The same frames into a ring of 4 images from two streams in turn, recorded once: the first blocks of a
    # frame start while the last blocks of the frame before drain (a frame is far too short to fill the GPU to its end).
    side = dev.stream()
    ring = [img] + [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(3)]
    for s_ in (st, side):
        ops.escape_time(s_, ring[1], p)
        s_.check()
    with st.record() as seq:
        st.fork_recording(side)
        for k in range(48):
            ops.escape_time(st if k % 2 == 0 else side, ring[k % 4], p)
    ms2 = time_launches(dev, st, lambda: seq.launch(), 5) / 48
    st.check()
    frame_line("mandelbrot 1080p, 48 frames recorded on two alternating streams, ring of 4", ms2, all(digest(r) == want for r in ring), "1080p, 2 streams, recorded")
    seq.close()
    for b in ring:
        b.close()

    # The reference program's own frame (fractal.py:7-25): 640 x 320 binary32 colour, |z| < 20, at most 50
    # steps, a new uniform every frame (fractal.py:30-31).  Such a frame costs a few microseconds of
    # arithmetic, so the launch is what is timed: plain launches against one recorded sequence.
    n_half, frames = 320, 256
    ring = [dev.empty((2 * n_half, n_half), np.float32, L.IMAGE) for _ in range(4)]  # field shape (2n, n): the real part follows the row index
    d = float(np.float32(2.0 / n_half))
    fparams = [ops.escape_params(L.JULIA, n_half, 2 * n_half, -1.0, -2.0, d, d, cr=-0.8, transposed=True,
                                 ci=float(np.float32(np.cos(np.float32(k * 0.03))) * np.float32(0.2)), max_iter=50,
                                 test=L.TEST_NORM_GE, bound=20.0, output=L.OUT_COLOR_F32, color_scale=0.02)
               for k in range(frames)]

    def run_frames(streams, params=None):
        for k, fp in enumerate(params or fparams):
            ops.escape_time(streams[k % len(streams)], ring[k % 4], fp)

    fparams_ring = []
    for fp in fparams:     # the same frames, each declared independent of the 3 before it (the ring has 4 slots)
        q = L.EscapeParams.from_buffer_copy(fp)
        q.flags |= 3 << 8
        fparams_ring.append(q)

    ms_plain = time_launches(dev, st, lambda: run_frames([st]), 5) / frames
    with st.record() as seq:
        run_frames([st])
    ms_seq = time_launches(dev, st, lambda: seq.launch(), 5) / frames
    with st.record() as seq2:
        st.fork_recording(side)
        run_frames([st, side])
    ms_seq2 = time_launches(dev, st, lambda: seq2.launch(), 5) / frames
    st.check()
    with st.record() as seq3:
        run_frames([st], fparams_ring)
    ms_seq3 = time_launches(dev, st, lambda: seq3.launch(), 5) / frames
    st.check()
    seq3.close()
    out.append({"workload": f"fractal.py frame 640x320 f32 colour max_iter=50, {frames} frames, a new uniform each", "kernel": "escape_time",
                "ms": min(ms_seq2, ms_seq3), "ms_plain_launches": ms_plain, "ms_recorded": ms_seq, "ms_recorded_two_streams": ms_seq2,
                "ms_recorded_one_stream_independent_launches": ms_seq3, "frames_per_s": 1e3 / min(ms_seq2, ms_seq3)})
    seq.close()
    seq2.close()
    side.close()
    for b in ring:
        b.close()
    return out


def compact(entries):
    """The workload lines once more, a few dozen characters each, for the end of the JSON line:
    [name, ms, fraction of the measured peak, fraction of the nominal peak, verified, worst error / tolerance]."""
    rows = []
    for e in entries:
        r = e.get("roofline", {})
        rows.append([e.get("short") or (e["kernel"] if e["kernel"] != "escape_time" else e["workload"][:28]), float(f"{e['ms']:.4g}"),
                     float(f"{r.get('frac', 0):.3g}"), float(f"{r.get('frac_of_nominal_8tbs', r.get('frac_of_nominal', 0)):.3g}"),
                     e.get("verified"), float(f"{e.get('max_err', 0):.2g}")])
    return rows


def round_floats(obj, digits=5):
    if isinstance(obj, float):
        return float(f"{obj:.{digits}g}")
    if isinstance(obj, dict):
        return {k: round_floats(v, digits) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [round_floats(v, digits) for v in obj]
    return obj


def run_only(args):
    """One kernel family at a reduced size, a few launches: the command ncu captures are taken from."""
    import torch

    import vernondsl_b200 as vd
    from vernondsl_b200 import _lib as L
    from vernondsl_b200 import ops

    dev = vd.Device(0)
    st = dev.stream()
    device = "cuda:0"
    gen = torch.Generator(device=device)
    gen.manual_seed(7)
    rn = lambda *shape: torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
    name, it = args.only, args.iters
    res = {"only": name, "scale": args.scale}
    if name == "fp32_probe":
        # what the FP32 pipe and the issue port do with scalar and with packed fma, alone and with integer work beside
        out = dev.empty(4, np.float32)
        per_thread, threads = 64 * 4000, dev.sm_count * 2048
        for variant, label in enumerate(("scalar fma", "packed fma.f32x2", "packed fma + 1 integer add each", "scalar fma + 1 integer add each")):
            ms = min(time_launches(dev, st, lambda: ops.fp32_probe(st, out, per_thread, threads, variant), 3, warmup=1) for _ in range(3))
            lane_fma = per_thread * threads * (2 if variant in (1, 2) else 1)
            res[label] = {"ms": ms, "T_lane_fma_per_s": lane_fma / (ms * 1e-3) / 1e12,
                          "instructions_per_clk_per_subpartition": per_thread * threads * (2 if variant >= 2 else 1) / 32 / (ms * 1e-3 * dev.sm_clock_khz * 1e3) / (dev.sm_count * 4)}
    elif name in ("escape_julia", "escape_mandelbrot"):
        side = max(256, int(16384 * args.scale) // 128 * 128)
        if name == "escape_julia":
            W = H = side
            dx, dy = ops.grid_steps(-1.6, 1.6, -1.6, 1.6, W, H)
            p = ops.escape_params(L.JULIA, W, H, -1.6, -1.6, dx, dy, cr=-0.8, ci=0.156, max_iter=4096)
        else:
            W, H = 1920, 1080
            dx, dy = ops.grid_steps(-2.5, 1.0, -1.0, 1.0, W, H)
            p = ops.escape_params(L.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=256)
        img = dev.empty((H, W), np.uint32, L.IMAGE)
        res["ms"] = time_launches(dev, st, lambda: ops.escape_time(st, img, p), it, warmup=1)
        res["shape"] = [H, W]
    elif name == "widen":
        # the receiving side of the image gather alone: uint16 rows of the peers -> the uint32 image, for a world of --world ranks
        W = H = max(2048, int(16384 * args.scale) // 2048 * 2048)
        world = max(2, args.world)
        wire, img = dev.empty((H, W), np.uint16, L.IMAGE), dev.empty((H, W), np.uint32, L.IMAGE)
        wire.fill(1)
        n_slabs = H // 128 // world
        res["ms"] = time_launches(dev, st, lambda: ops.widen_rows_u16(st, wire, img, W, H, 128, world, 0, 0, n_slabs), it, warmup=2)
        moved = (world - 1) * n_slabs * 128 * W * 6
        res["world"], res["gbs"] = world, moved / res["ms"] / 1e6
    elif name in ("escape_split", "escape_beside"):
        from vernondsl_b200 import partition

        W = H = max(2048, int(16384 * args.scale) // 2048 * 2048)
        dx, dy = ops.grid_steps(-1.6, 1.6, -1.6, 1.6, W, H)
        img = dev.empty((H, W), np.uint32, L.IMAGE)
        world = max(1, args.world)
        plan = partition.plan_image(H, world, 0, L.PART_CYCLIC, 128)        # rank 0's share of a world of that size
        base = ops.escape_params(L.JULIA, W, H, -1.6, -1.6, dx, dy, cr=-0.8, ci=0.156, max_iter=4096, partition=plan.part)
        st2 = dev.stream()
        res["shape"], res["world"] = [H, W], world
        if name == "escape_split":
            # what a step costs when the rank's rows go out in G launches (combs of slabs), on one stream and on two in turn
            def launches(groups, streams):
                def fn():
                    e = dev.event()
                    e.record(st)
                    st2.wait(e)
                    for k, ((first, step_, count), _) in enumerate(partition.comb_groups(plan, groups)):
                        gp = copy.copy(base)
                        gp.chunk_first, gp.chunk_step, gp.chunk_count = first, step_, count
                        ops.escape_time(streams[k % len(streams)], img, gp)
                    e2 = dev.event()
                    e2.record(st2)
                    st.wait(e2)
                    e.close(); e2.close()   # destruction is deferred until the recorded work has passed
                return fn
            res["ms_one_launch"] = time_launches(dev, st, launches(1, [st]), it, warmup=2)
            for g in (2, 4, 8):
                res[f"ms_{g}_launches_one_stream"] = time_launches(dev, st, launches(g, [st]), it, warmup=2)
                res[f"ms_{g}_launches_two_streams"] = time_launches(dev, st, launches(g, [st, st2]), it, warmup=2)
        else:
            # does a small memory-bound kernel on another stream run while the escape-time kernel runs?
            wire = dev.empty((H, W), np.uint16, L.IMAGE)
            img2 = dev.empty((H, W), np.uint32, L.IMAGE)
            flags = dev.empty((8,), np.uint32, L.STORAGE_BUFFER)
            ops.escape_time(st, img, base, wire=wire)
            ops.widen_rows_u16(st2, wire, img2, W, H, 128, 2, 0, 0, 8)
            dev.synchronize()
            for order in ("escape_first", "helpers_first"):
                e0, e_esc, e_sig, e_wid = (dev.event() for _ in range(4))
                dev.synchronize()
                e0.record(st)
                st2.wait(e0)

                def helpers():
                    ops.gather_signal(st2, [flags], 2, 1, 1)
                    e_sig.record(st2)
                    ops.widen_rows_u16(st2, wire, img2, W, H, 128, 2, 0, 0, 8)
                    e_wid.record(st2)

                def escape():
                    ops.escape_time(st, img, base)
                    e_esc.record(st)

                (escape(), helpers()) if order == "escape_first" else (helpers(), escape())
                dev.synchronize()
                res[order] = {"escape_done_ms": e0.elapsed_ms(e_esc), "one_warp_kernel_done_ms": e0.elapsed_ms(e_sig),
                              "widen_done_ms": e0.elapsed_ms(e_wid)}
            e0, e1 = dev.event(), dev.event()
            e0.record(st2)
            ops.widen_rows_u16(st2, wire, img2, W, H, 128, 2, 0, 0, 8)
            e1.record(st2)
            e1.synchronize()
            res["widen_alone_ms"] = e0.elapsed_ms(e1)
        st2.check()
    elif name in ("fused_map", "map_tape"):
        n = int((1 << 28) * args.scale) // 4096 * 4096
        a, x, y, o = rn(n), rn(n), rn(n), torch.empty(n, device=device)
        A, X, Y, O = (dev.wrap_tensor(t) for t in (a, x, y, o))
        if name == "fused_map":
            fn = lambda: ops.fused_map(st, A, X, Y, O, n)
        else:
            t = ops.Tape(3)
            u = t.op("fma", t.input(0), t.input(1), t.input(2))
            e = t.op("exp", t.op("mul", t.op("mul", t.const(-0.5), t.input(1)), t.input(1)))
            q = t.op("sqrt", t.op("add", t.op("abs", t.input(2)), t.const(1e-3)))
            t.output(t.op("fma", t.op("tanh", u), e, q))
            fn = lambda: ops.map_tape(st, t, [A, X, Y], [O], n // 4096, 4096)
        res["ms"] = time_launches(dev, st, fn, it, warmup=1)
        res["gbs"] = 16 * n / res["ms"] / 1e6
    elif name.startswith("row_"):
        R, Cc = max(8, int(65536 * args.scale)), 4096
        m, sm = rn(R, Cc) * 2, torch.empty((R, Cc), device=device)
        rs, rm = torch.empty(R, device=device), torch.empty(R, device=device)
        M, SM, RS, RM = (dev.wrap_tensor(t) for t in (m, sm, rs, rm))
        fn = {"row_sum": lambda: ops.row_sum(st, M, RS, R, Cc), "row_max": lambda: ops.row_max(st, M, RM, R, Cc),
              "row_softmax": lambda: ops.row_softmax(st, M, SM, R, Cc),
              "row_stats_softmax": lambda: ops.row_stats_softmax(st, M, RS, RM, SM, R, Cc)}[name]
        res["ms"] = time_launches(dev, st, fn, it, warmup=1)
        res["gbs"] = (8 if "softmax" in name else 4) * R * Cc / res["ms"] / 1e6
    elif name in ("mse_fwd", "mse_bwd"):
        R, Cc = max(8, int(32768 * args.scale)), 4096
        Wt, xt, tt, bt = rn(R, Cc), rn(R, Cc), rn(R, Cc), rn(Cc)
        dWt, dxt, dbt, lt = torch.empty_like(Wt), torch.empty_like(Wt), torch.empty(Cc, device=device), torch.empty(4, device=device)
        bW, bx, bb, bt_, bdW, bdx, bdb, bl = (dev.wrap_tensor(t) for t in (Wt, xt, bt, tt, dWt, dxt, dbt, lt))
        fn = (lambda: ops.mse_tanh_fwd(st, bW, bx, bb, bt_, bl, R, Cc)) if name == "mse_fwd" else \
            (lambda: ops.mse_tanh_bwd(st, bW, bx, bb, bt_, bdW, bdx, bdb, R, Cc))
        res["ms"] = time_launches(dev, st, fn, it, warmup=1)
        res["gbs"] = (12 if name == "mse_fwd" else 20) * R * Cc / res["ms"] / 1e6
    else:
        raise SystemExit(f"unknown --only {name}")
    st.check()
    print(json.dumps(res), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, help="run one kernel family at reduced size (for profiling) and exit")
    ap.add_argument("--scale", type=float, default=0.25, help="with --only: fraction of the full workload size")
    ap.add_argument("--iters", type=int, default=3, help="with --only: timed launches")
    ap.add_argument("--world", type=int, default=1, help="with --only escape_split/escape_beside: time rank 0's share of a world of this size")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workloads", default="all", choices=["all", "main"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", default="push16", choices=["push16", "pull16", "p2p", "nccl"],
                    help="N > 1: how the image is gathered.  push16: the library's own exchange (vrhi_exchange_*): uint16 counts stored "
                         "into the peers by a small kernel, no collective library; pull16: every rank reads its peers' uint16 counts over NVLink and "
                         "widens them in the same kernel; "
                         "p2p: uint32 rows pushed by the copy engines; nccl: NCCL all-gather")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return
    if args.only:
        run_only(args)
        return

    # NCCL prints its version banner on stdout; the contract is ONE JSON line there.  Everything
    # a library writes to fd 1 goes to stderr from here on; the JSON line uses the saved descriptor.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    import vernondsl_b200 as vd
    from vernondsl_b200 import _lib as L
    from vernondsl_b200 import group, ops, partition

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")

    dev = vd.Device(local)
    tstream = torch.cuda.Stream(device=local)
    st = dev.wrap_stream(tstream.cuda_stream)
    hbm_peak, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # FP32 issue-rate probe (FFMA chains): the denominator of the escape-time roofline
    probe_out = dev.empty(4, np.float32)
    per_thread = 64 * 4000
    threads = dev.sm_count * 2048
    probe_ms = min(time_launches(dev, st, lambda: ops.fp32_probe(st, probe_out, per_thread, threads), 3, warmup=1) for _ in range(3))
    fp32_peak = per_thread * threads / (probe_ms * 1e-3) / 1e9  # G lane-instructions / s
    fp32_nominal = dev.sm_count * 128 * dev.sm_clock_khz * 1e3 / 1e9

    J = JULIA
    W, H = J["W"], J["H"]
    dx, dy = ops.grid_steps(J["x0"], J["x1"], J["y0"], J["y1"], W, H)
    plan = partition.plan_image(H, world, rank, L.PART_CYCLIC, 128)
    # the image is allocated by the library (so that peers can map it); torch sees the same memory
    image = dev.empty((H, W), np.uint32, L.IMAGE)
    image.fill(0)
    image_t = image.as_tensor(np.uint32, (H, W))
    params = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=J["max_iter"],
                               partition=plan.part if world > 1 else None)
    total_iters = golden_total()

    def compute():
        ops.escape_time(st, image, params)

    # With N > 1 a step is pipelined: the rank's chunks are computed in GROUPS launches, and the
    # in-place all-gather of the slabs a launch completed runs on a second stream while the next
    # launch computes.  The step ends when the last gather has finished.
    # launches per step; finished slabs are exchanged while the next launch computes.  More groups shorten the last,
    # exposed push; every launch adds ramp-up and drain, most of which the two alternating compute streams hide.
    # measured on B200 (ms per step): 2 ranks 1.35 with 6 groups (1.36 with 4); 4 ranks 1.02 with 4 (1.03 with 6, 1.05 with 3);
    # 8 ranks 1.11 with 2 (1.17 with 4): with seven peers a group's seven copies want to be large
    GROUPS = int(os.environ.get("VRHI_BENCH_GROUPS", "6" if world <= 2 else "4" if world <= 4 else "2"))
    COMM_STREAMS = 2 if (os.environ.get("VRHI_BENCH_COMM_STREAMS", "1") == "2" and world > 2) else 1   # pushes to odd and even peers on two streams
    # Group g takes slabs g, g+GROUPS, g+2*GROUPS, ...: every group is a thin comb over the whole image, so the
    # groups cost the same although the rows near the set cost far more than the rows at the edges.
    exchange, grp = None, None
    n_slabs = plan.part.chunk_count
    group_params, group_slabs = [], []
    if world > 1:
        for (first, step_, count), slabs in partition.comb_groups(plan, GROUPS):
            gp = copy.copy(params)
            gp.chunk_first, gp.chunk_step, gp.chunk_count = first, step_, count
            group_params.append(gp)
            group_slabs.append(slabs)
        comm_stream = torch.cuda.Stream(device=local)
        comm_st = dev.wrap_stream(comm_stream.cuda_stream)
        if COMM_STREAMS == 2:
            comm_stream2 = torch.cuda.Stream(device=local)
            comm_st2 = dev.wrap_stream(comm_stream2.cuda_stream)
        exchange = None
        try:
            grp = group.Group(dev, world, rank, group.torch_allgather())   # bootstrap over the process group; the data path is the library's
        except Exception as exc:  # no peer mapping on this box
            print(f"vrhi_group unavailable ({exc}); using torch.distributed for the exchange steps", file=sys.stderr)
            grp = None
        if args.gather != "nccl" and grp is not None:
            try:
                if args.gather == "push16":
                    exchange = grp.image_exchange(image, W, H, 128)
                elif args.gather == "pull16":
                    exchange = partition.PullImageExchange(dev, image, plan, W, groups=len(group_params))
                    sig_stream = torch.cuda.Stream(device=local)
                    sig_st = dev.wrap_stream(sig_stream.cuda_stream)
                else:
                    exchange = partition.PeerImageExchange(dev, image, plan, W * 4)
            except Exception as exc:  # no peer mapping on this box: fall back to the NCCL gather
                print(f"peer exchange unavailable ({exc}); using the NCCL all-gather", file=sys.stderr)

    TWO_COMPUTE_STREAMS = world > 1 and os.environ.get("VRHI_BENCH_COMPUTE_STREAMS", "2") == "2"
    if TWO_COMPUTE_STREAMS:
        tstream2 = torch.cuda.Stream(device=local)
        st2 = dev.wrap_stream(tstream2.cuda_stream)
    pulling = isinstance(exchange, partition.PullImageExchange)
    native = isinstance(exchange, group.Exchange)
    trace = []   # (label, event) of one extra, untimed step when VRHI_BENCH_TRACE is set: where a step's time goes
    TRACING = [False]

    def mark(label, stream):
        if TRACING[0]:
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            trace.append((label, e))

    def step():
        if world == 1:
            compute()
            return
        works = []
        mark("start", tstream)
        if native:
            # the whole exchange is the library's: publish after each group's launch, complete at the end of the step
            wire, byte_plane = exchange.planes
            if TWO_COMPUTE_STREAMS:
                tstream2.wait_stream(tstream)
            for gi, (gp, slabs) in enumerate(zip(group_params, group_slabs)):
                cs_t, cs = (tstream2, st2) if (TWO_COMPUTE_STREAMS and gi % 2) else (tstream, st)
                ops.escape_time(cs, image, gp, wire=wire, byte_plane=byte_plane)
                mark(f"computed {gi}", cs_t)
                exchange.publish(cs, slabs)
            if TWO_COMPUTE_STREAMS:
                tstream.wait_stream(tstream2)
            exchange.complete(st)
            mark("exchange complete", tstream)
            return
        wire = exchange.wire if pulling else None
        if TWO_COMPUTE_STREAMS:
            tstream2.wait_stream(tstream)
        for gi, (gp, slabs) in enumerate(zip(group_params, group_slabs)):
            # launches alternate between two streams: the first blocks of a group start while the last blocks of
            # the group before drain (each launch otherwise pays ~60 us of ramp-up and drain by itself)
            cs_t, cs = (tstream2, st2) if (TWO_COMPUTE_STREAMS and gi % 2) else (tstream, st)
            ops.escape_time(cs, image, gp, wire=wire)
            mark(f"computed {gi}", cs_t)
            ev = torch.cuda.Event()
            ev.record(cs_t)
            comm_stream.wait_event(ev)
            if pulling:
                # tell the peers this group is ready (own stream: the next group's kernel is not held up), then
                # fetch their rows of the same group: remote uint16 loads over NVLink, widened into the image
                sig_stream.wait_event(ev)
                exchange.signal(sig_st, gi)
                exchange.pull(comm_st, gi, slabs)
                mark(f"pulled {gi}", comm_stream)
            elif exchange is not None:
                # copy engines: the pushes overlap the next group's kernel
                if COMM_STREAMS == 2:
                    comm_stream2.wait_event(ev)
                    exchange.push([comm_st if k % 2 == 0 else comm_st2 for k in range(world - 1)], slabs)
                else:
                    exchange.push(comm_st, slabs)
                mark(f"pushed {gi}", comm_stream)
            else:
                with torch.cuda.stream(comm_stream):
                    works += partition.all_gather_image(image_t, plan, async_op=True, slabs=slabs)
        if TWO_COMPUTE_STREAMS:
            tstream.wait_stream(tstream2)
        if pulling:
            tstream.wait_stream(sig_stream)
            tstream.wait_stream(comm_stream)
            exchange.next_step()
        elif exchange is not None:
            if COMM_STREAMS == 2:
                comm_stream.wait_stream(comm_stream2)
            exchange.finish(comm_stream)
            mark("exchange complete", comm_stream)
            tstream.wait_stream(comm_stream)
            if COMM_STREAMS == 2:
                tstream.wait_stream(comm_stream2)
        else:
            with torch.cuda.stream(tstream):
                for w in works:
                    w.wait()   # the compute stream waits for the gathers: the step is complete after this

    EXCHANGE_NOTE = ("none" if world == 1 else
                     "vrhi_exchange (C ABI, no collective library): the copy engines move every rank's rows into its peers while the next group "
                     "computes (uint16 counts at 2 ranks; from 3 ranks on a byte plane, counts of 255 and more fetched from the owner), "
                     "sequence flags with bounded device waits, widened on arrival" if native else
                     "no collective: each rank reads its peers' rows as uint16 out of their memory over NVLink and widens them into "
                     "its uint32 image in one kernel, group by group while later groups compute; readiness flags with bounded device waits" if pulling else
                     "image chunks pushed into every peer's image by strided peer copies (copy engines over NVLink), overlapped with "
                     "compute; one 4-byte NCCL all-reduce orders completion" if exchange is not None else
                     "in-place NCCL all-gather of the image each step, overlapped with compute")

    def timed(fn, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(tstream):
            e0.record(tstream)
            for _ in range(k):
                fn()
            e1.record(tstream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=f"cuda:{local}")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # clocks are sampled from the first warm-up step to the end of the timed steps, and on through
    # ~0.3 s more of the same steps (the timed region alone is tens of milliseconds: too short for
    # nvidia-smi to see more than one sample of it)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    def count_launches():
        # kernels of this library on every stream a step uses (compute, and the arrival or pull streams)
        n = st.launch_count()
        if native:
            n += exchange.launch_count()
        if world > 1:
            n += comm_st.launch_count()
            if TWO_COMPUTE_STREAMS:
                n += st2.launch_count()
            if pulling:
                n += sig_st.launch_count()
        return n

    launches0 = count_launches()
    total_ms = timed(step, args.steps)
    launches = count_launches() - launches0
    if native:
        exchange.check()   # raises if a device-side wait gave up (a peer never arrived); with VRHI_EXCHANGE_TRACE=1 prints the last step's timeline
    if world > 1 and os.environ.get("VRHI_BENCH_TRACE"):
        barrier()
        TRACING[0] = True
        with torch.cuda.stream(tstream):
            step()
        TRACING[0] = False
        torch.cuda.synchronize()
        print(f"rank {rank} step timeline (ms after start): " + ", ".join(f"{lab} {trace[0][1].elapsed_time(e):.3f}" for lab, e in trace[1:]), file=sys.stderr)
    t_hold = time.perf_counter()
    while time.perf_counter() - t_hold < 0.3:
        step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = total_iters / (ms_per_step * 1e-3) / 1e9

    # the image every rank now holds must be the oracle's, bit for bit (exact integer digest)
    got_sum = int(image_t.sum(dtype=torch.int64).item())
    idx = torch.arange(1, H * W + 1, device=f"cuda:{local}", dtype=torch.int64)
    got_wsum = int((image_t.view(-1).to(torch.int64) * idx).sum().item()) & 0xFFFFFFFFFFFFFFFF
    del idx
    g = np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))
    verified = [got_sum, got_wsum] == [int(v) for v in g["julia_16k_digest"]]

    compute_ms = timed(compute, args.steps) / args.steps if world > 1 else ms_per_step
    compute_value = total_iters / (compute_ms * 1e-3) / 1e9

    # the contracted arithmetic mode, reported separately with its pixel-mismatch fraction
    fast_mode = None
    if world == 1:
        exact_img = image_t.clone()
        fparams = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=J["max_iter"], mode=L.FAST)
        fast_fn = lambda: ops.escape_time(st, image, fparams)
        for _ in range(3):
            fast_fn()
        fast_ms = timed(fast_fn, args.steps) / args.steps
        fast_iters = int(image_t.sum(dtype=torch.int64).item())
        mismatch = float((image_t != exact_img).sum().item()) / (W * H)
        fast_mode = {"value": fast_iters / (fast_ms * 1e-3) / 1e9, "unit": "Gpixel-iters/s", "ms_per_step": fast_ms,
                     "pixel_mismatch_fraction_vs_exact": mismatch, "sum_of_counts": fast_iters,
                     "note": "multiply-adds fused: its own rounding sequence, not bit-comparable with the exact mode"}
        del exact_img
        compute()  # leave the exact image in place for the end-to-end leg

    # end to end through the public API: the result lands in pinned host memory every step
    chunks = plan.chunks() if world > 1 else [(0, H)]
    host = vd.PinnedArray((sum(n for _, n in chunks), W), np.uint32)

    # The rank's rows are computed in E2E_GROUPS launches; the download of a finished group runs on a
    # copy stream while the next group computes, so a step costs about max(compute, PCIe transfer).
    E2E_GROUPS = 8
    own = ops.partition_rows(H, world, rank, L.PART_CYCLIC, 128)
    e2e_groups = []
    row_cursor = 0
    for gidx in range(E2E_GROUPS):
        k0, k1 = own.chunk_count * gidx // E2E_GROUPS, own.chunk_count * (gidx + 1) // E2E_GROUPS
        if k1 == k0:
            continue
        gp = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=J["max_iter"], partition=own)
        gp.chunk_first = own.chunk_first + k0 * own.chunk_step
        gp.chunk_count = k1 - k0
        spans = []
        for k in range(k0, k1):
            r0 = (own.chunk_first + k * own.chunk_step) * own.chunk_rows
            n = min(H, r0 + own.chunk_rows) - r0
            if spans and world == 1 and spans[-1][0] + spans[-1][1] == r0:
                spans[-1] = (spans[-1][0], spans[-1][1] + n, spans[-1][2])   # contiguous on one GPU: one copy
            else:
                spans.append((r0, n, row_cursor))
            row_cursor += n
        e2e_groups.append((gp, spans))
    copy_tstream = torch.cuda.Stream(device=local)
    copy_st = dev.wrap_stream(copy_tstream.cuda_stream)

    def e2e_step():
        for gp, spans in e2e_groups:
            ops.escape_time(st, image, gp)
            ev = torch.cuda.Event()
            ev.record(tstream)
            copy_tstream.wait_event(ev)
            for r0, n, dst_row in spans:
                image.download(host.array[dst_row:dst_row + n], offset=r0 * W * 4, stream=copy_st)
        copy_st.synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=f"cuda:{local}", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = total_iters * e2e_steps / float(e2e_s.item()) / 1e9
    d2h = sum(n for _, n in chunks) * W * 4
    host.close()

    # The same end-to-end step with the counts delivered as uint16 (VRHI_OUT_COUNT_U16; max_iter = 4096 fits): the
    # step is bound by the device-to-host link, so half the bytes is close to twice the rate.  Extra line, N = 1 only.
    e2e_u16 = None
    if world == 1:
        image16 = dev.empty((H, W), np.uint16, L.IMAGE)
        host16 = vd.PinnedArray((H, W), np.uint16)
        groups16 = []
        for gp, spans in e2e_groups:
            gp16 = copy.copy(gp)
            gp16.output = L.OUT_COUNT_U16
            groups16.append((gp16, spans))

        def e2e16_step():
            for gp16, spans in groups16:
                ops.escape_time(st, image16, gp16)
                ev = torch.cuda.Event()
                ev.record(tstream)
                copy_tstream.wait_event(ev)
                for r0, n, dst_row in spans:
                    image16.download(host16.array[dst_row:dst_row + n], offset=r0 * W * 2, stream=copy_st)
            copy_st.synchronize()

        for _ in range(2):
            e2e16_step()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e16_step()
        secs = time.perf_counter() - t0
        ok16 = bool(int(host16.array.astype(np.uint64).sum()) == total_iters)
        e2e_u16 = {"value": total_iters * e2e_steps / secs / 1e9, "unit": "Gpixel-iters/s", "d2h_bytes_per_step": H * W * 2,
                   "sum_of_counts_matches": ok16}
        host16.close()
        image16.close()

    # the other workloads: frame-sized escape-time launches (one GPU), and the HBM-bound map / row / backward
    # workloads at their full shapes, split along the leading axis at N > 1, each checked against the oracle
    others = []
    barrier()
    if exchange is not None:
        exchange.close()   # peers hold mappings of this rank's buffers: unmap them before anything is freed
        exchange = None
        barrier()
    if args.workloads == "all":
        image.close()
        del image_t
        torch.cuda.empty_cache()
        if world == 1:
            others += frame_workloads(dev, st, torch, fp32_peak, fp32_nominal)
        others += hbm_workloads(dev, st, torch, rank, world, hbm_peak, peak_kind, grp)

    if rank == 0:
        achieved = OPS_PER_ITER * total_iters / (compute_ms * 1e-3) / 1e9 / world  # per GPU
        line = {
            "metric": "Gpixel-iters/s", "value": value, "unit": "Gpixel-iters/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "partition": f"cyclic 128-row chunks over {world} rank(s)",
                       "collective": EXCHANGE_NOTE,
                       "l2": "no inputs; the 1 GiB output image written each step exceeds L2 (126 MB)"},
            "verified_bit_exact": verified,
            "compute_only": {"value": compute_value, "ms_per_step": compute_ms},
            "roofline": {"bound": "fp32", "achieved": achieved, "peak": fp32_peak, "unit": "Gop/s", "frac": achieved / fp32_peak,
                         # DRAM bytes one GPU moves per step: the rows it computes, once (an ncu capture of the 8192^2
                         # image showed 210.6 MB written for 268.4 MB of image, the rest still in L2, and 0.8 MB read)
                         "traffic": float(H * W * 4 // world), "traffic_source": "bytes of the rows this GPU writes; not measured in this run",
                         "peak_kind": "FFMA-chain probe in this run (lane-instructions/s)",
                         "peak_nominal": fp32_nominal, "frac_of_nominal": achieved / fp32_nominal,
                         "algorithmic": f"{OPS_PER_ITER} f32 ops per pixel-iteration x {total_iters} iterations per image, per GPU"},
            "e2e": {"value": e2e_value, "unit": "Gpixel-iters/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches), "clocks": clocks, "fast_mode": fast_mode,
        }
        if e2e_u16 is not None:
            line["e2e_uint16_result"] = e2e_u16
        if world == 1 and not args.no_cpu_baseline:
            import oracle

            oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
            t0 = time.perf_counter()
            _, tot = oracle.escape_time(oracle.JULIA, W, H, J["x0"], J["y0"], dx, dy, J["cr"], J["ci"], J["max_iter"], want_image=False)
            secs = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": tot / secs / 1e9, "unit": "Gpixel-iters/s", "cores": oracle.num_threads(), "kind": "port",
                                    "sample": "the whole 16384x16384 image, once"}
        if others:
            line["other_workloads"] = others
            # last key, short: [kernel or workload, ms, fraction of the measured peak, of the nominal peak, verified, worst error / tolerance]
            line["summary"] = {"headline": [float(f"{ms_per_step:.4g}"), float(f"{achieved / fp32_peak:.3g}"), float(f"{achieved / fp32_nominal:.3g}"), verified],
                               "others": compact(others)}
        os.write(json_fd, (json.dumps(round_floats(line), separators=(",", ":")) + "\n").encode())
    barrier()
    if exchange is not None:
        exchange.close()
    if grp is not None:
        grp.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
