"""CPU: the checks the benchmark applies to its full-shape workloads are not vacuous.

bench.check_fused_map / check_rows / check_mse decide the `verified` field of every workload line.
Here they run on small CPU tensors: a correct result must pass, and a result with one wrong value
in a place the check looks at (a window's tail, a sampled row, one column of db) must fail."""
import numpy as np
import pytest

import bench
import oracle

torch = pytest.importorskip("torch")


def test_fused_map_check_accepts_the_oracle_and_rejects_a_wrong_tail():
    rng = np.random.default_rng(5)
    n = 200_000
    a, x, y = (rng.uniform(-1, 1, n).astype(np.float32), rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32))
    out = oracle.fused_map(a, x, y)
    ta, tx, ty, to = (torch.from_numpy(v) for v in (a, x, y, out.copy()))
    ok, worst = bench.check_fused_map(ta, tx, ty, to)
    assert ok and worst <= 1.0
    to[n - 1] += 1e-3          # the very last element: an unwritten or mis-indexed tail would look like this
    ok, worst = bench.check_fused_map(ta, tx, ty, to)
    assert not ok and worst > 1.0
    to = torch.from_numpy(out.copy())
    to[0] = 0.0                # and the very first
    assert not bench.check_fused_map(ta, tx, ty, to)[0]


def test_row_check_accepts_the_oracle_and_rejects_a_wrong_row():
    m = (2.0 * np.random.default_rng(6).standard_normal((300, 512))).astype(np.float32)
    tm = torch.from_numpy(m)
    rs, rm, sm = (torch.from_numpy(f(m).copy()) for f in (oracle.row_sum, oracle.row_max, oracle.row_softmax))
    assert bench.check_rows(tm, rs, rm, sm)[0]
    bad = sm.clone()
    bad[299, 17] *= 1.001      # the last row is always among the sampled ones
    assert not bench.check_rows(tm, softmax=bad)[0]
    bad = rm.clone()
    bad[0] += 1.0              # so is the first
    assert not bench.check_rows(tm, row_max=bad)[0]
    bad = rs.clone()
    bad[299] += 1.0
    assert not bench.check_rows(tm, row_sum=bad)[0]


def test_backward_check_accepts_the_oracle_and_rejects_a_wrong_column_sum():
    rng = np.random.default_rng(7)
    R, Cc = 400, 256
    W, x, t = (rng.standard_normal((R, Cc)).astype(np.float32) for _ in range(3))
    b = rng.standard_normal(Cc).astype(np.float32)
    dW, dx, db = oracle.mse_tanh_bwd(W, x, b, t)
    loss = oracle.mse_tanh_fwd(W, x, b, t)
    tW, tx, tb, tt = (torch.from_numpy(v) for v in (W, x, b, t))
    tdW, tdx, tdb = torch.from_numpy(dW.copy()), torch.from_numpy(dx.copy()), torch.from_numpy(db.astype(np.float32))
    denom = float(R * Cc)
    assert bench.check_mse(tW, tx, tb, tt, denom, tdW, tdx, 0, db=tdb, loss=loss)[0]
    bad = tdb.clone()
    bad[200] *= 1.01           # one column of db: only a check of ALL of db sees it
    assert not bench.check_mse(tW, tx, tb, tt, denom, db=bad)[0]
    assert not bench.check_mse(tW, tx, tb, tt, denom, loss=loss * 1.0001)[0]
    # a row shard: rows 100..299 of the problem, checked against the same rows of the whole
    assert bench.check_mse(tW, tx, tb, tt, denom, tdW[100:300], tdx[100:300], 100)[0]
    assert not bench.check_mse(tW, tx, tb, tt, denom, tdW[101:301], tdx[101:301], 100)[0]   # shifted by one row: wrong rows


def test_compact_summary_carries_every_line():
    lines = [{"workload": "w", "kernel": "k", "ms": 0.123456, "roofline": {"frac": 1.0456, "frac_of_nominal_8tbs": 0.8561}, "verified": True, "max_err": 0.01234},
             {"workload": "mandelbrot frames and more text", "kernel": "escape_time", "ms": 0.05, "roofline": {"frac": 0.5, "frac_of_nominal": 0.47}, "verified": True}]
    rows = bench.compact(lines)
    assert rows[0] == ["k", 0.1235, 1.05, 0.856, True, 0.012]
    assert rows[1][0].startswith("mandelbrot") and rows[1][3] == 0.47
    assert bench.round_floats({"a": 1.23456789, "b": [2.000001, "s"], "c": 3}) == {"a": 1.2346, "b": [2.0, "s"], "c": 3}


def test_the_summary_of_a_default_run_fits_a_1500_character_tail():
    """Whoever keeps only the end of the benchmark's line must still find every workload in it: the summary is the
    last key, and with the names a default single-GPU run produces and the widest numbers it can print it stays
    well under 1500 characters."""
    import json

    names = ["1080p, 1 stream, 1 image", "1080p, 1 stream, ring of 4", "1080p, 1 stream, ring of 8, recorded", "1080p, 2 streams, recorded",
             "fractal.py frame 640x320 f32", "fused_map", "map_tape (compiled at first use)", "map_tape (interpreted)", "row_sum", "row_max",
             "row_softmax", "row_stats_softmax", "mse_tanh_fwd", "mse_tanh_bwd", "graph: 1 kernels", "graph: 3 kernels"]
    lines = [{"workload": n, "short": n if n[0] in "1f" and n != "fused_map" else None, "kernel": "escape_time" if n[0] == "1" or n.startswith("fractal") else n,
              "ms": 0.0123456, "roofline": {"frac": 0.98765, "frac_of_nominal_8tbs": 0.87654}, "verified": False, "max_err": 0.00098765} for n in names]
    rows = bench.compact(lines)
    assert [r[0] for r in rows] == names
    tail = json.dumps({"summary": {"headline": [2.123, 0.752, 0.714, False], "others": rows}})
    assert len(tail) < 1400, len(tail)
