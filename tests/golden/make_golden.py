"""Regenerates tests/golden/golden.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference project holds no golden vector for this path (parity is unpinned by it), so these
fixtures freeze the oracle's own output: small count images, exact digests of the two full-size
escape-time workloads, and float vectors for the map / row / gradient operators.  The GPU tests
compare against them without running the oracle at full size, and the CPU tests check that the
oracle still reproduces them.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

import oracle  # noqa: E402

WORKLOADS = {
    # name: kind, W, H, x0, x1, y0, y1, cr, ci, max_iter
    "mandelbrot_1080p": (oracle.MANDELBROT, 1920, 1080, -2.5, 1.0, -1.0, 1.0, 0.0, 0.0, 256),
    "julia_16k": (oracle.JULIA, 16384, 16384, -1.6, 1.6, -1.6, 1.6, -0.8, 0.156, 4096),
    "julia_512": (oracle.JULIA, 512, 512, -1.6, 1.6, -1.6, 1.6, -0.8, 0.156, 4096),
    "mandelbrot_ragged": (oracle.MANDELBROT, 157, 43, -2.5, 1.0, -1.0, 1.0, 0.0, 0.0, 300),
}


def workload_image(name, want_image=True):
    kind, W, H, x0, x1, y0, y1, cr, ci, mi = WORKLOADS[name]
    dx, dy = oracle.grid_steps(x0, x1, y0, y1, W, H)
    return oracle.escape_time(kind, W, H, x0, y0, dx, dy, cr, ci, mi, want_image=want_image)


def main():
    out = {}
    for name in WORKLOADS:
        img, total = workload_image(name)
        s, w = oracle.digest_u32(img)
        assert s == total
        out[f"{name}_digest"] = np.array([s, w], dtype=np.uint64)
        if img.size <= 512 * 512:
            out[f"{name}_counts"] = img.astype(np.uint16 if img.max() < 65536 else np.uint32)
        else:
            out[f"{name}_rows"] = np.array([0, img.shape[0] // 3, img.shape[0] // 2, img.shape[0] - 1], dtype=np.int64)
            out[f"{name}_row_counts"] = img[out[f"{name}_rows"]].astype(np.uint16)
        print(name, "sum", s, "wsum", w)

    rng = np.random.default_rng(1001)
    n = 4099  # not a multiple of 4
    a = rng.uniform(-1, 1, n).astype(np.float32)
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    out["map_a"], out["map_x"], out["map_y"] = a, x, y
    out["map_out"] = oracle.fused_map(a, x, y)

    m = (2.0 * rng.standard_normal((9, 260))).astype(np.float32)
    out["rows_in"] = m
    out["rows_sum"], out["rows_max"], out["rows_softmax"] = oracle.row_sum(m), oracle.row_max(m), oracle.row_softmax(m)

    R, Cc = 13, 36
    W_ = rng.standard_normal((R, Cc)).astype(np.float32)
    x_ = rng.standard_normal((R, Cc)).astype(np.float32)
    t_ = rng.standard_normal((R, Cc)).astype(np.float32)
    b_ = rng.standard_normal(Cc).astype(np.float32)
    dW, dx, db = oracle.mse_tanh_bwd(W_, x_, b_, t_)
    out.update(mse_W=W_, mse_x=x_, mse_t=t_, mse_b=b_, mse_dW=dW, mse_dx=dx, mse_db=db,
               mse_loss=np.array([oracle.mse_tanh_fwd(W_, x_, b_, t_)], dtype=np.float64))
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"))


if __name__ == "__main__":
    main()
