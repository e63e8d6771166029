"""Second, independently written CPU statement of the hot path -- TEST INFRASTRUCTURE.

Vectorised numpy (binary32 arithmetic without fused multiply-add, which numpy never uses for
separate ``*`` and ``+``) for the escape-time map, and float64 numpy for the floating-point
operators.  It exists only so that the C oracle is not its own witness: the tests require the two
to agree bit for bit on counts and to float64 round-off on the rest.

Loop rules follow fractal.py:18-25: test first, then update, count the updates.
"""
from __future__ import annotations

import numpy as np

f32 = np.float32


def escape_time(kind, width, height, x0, y0, dx, dy, cr=0.0, ci=0.0, max_iter=256,
                test=0, bound=4.0, rows=None):
    """kind 0 = Mandelbrot (z0 = 0, c = pixel); kind 1 = Julia (z0 = pixel, c = (cr, ci)).
    test 0: stop when zr*zr + zi*zi > bound; test 1: stop unless sqrt(zr*zr + zi*zi) < bound."""
    rows = np.arange(height) if rows is None else np.asarray(rows)
    i = np.arange(width, dtype=np.float32)
    j = rows.astype(np.float32)
    x = (f32(x0) + i * f32(dx)).astype(np.float32)
    y = (f32(y0) + j * f32(dy)).astype(np.float32)
    X, Y = np.meshgrid(x, y)          # [rows, width]
    if kind == 0:
        zr = np.zeros_like(X)
        zi = np.zeros_like(X)
        Cr, Ci = X.copy(), Y.copy()
    else:
        zr, zi = X.copy(), Y.copy()
        Cr = np.full_like(X, f32(cr))
        Ci = np.full_like(X, f32(ci))
    count = np.zeros(X.shape, dtype=np.uint32)
    live = np.ones(X.shape, dtype=bool)
    bound = f32(bound)
    with np.errstate(over="ignore", invalid="ignore"):
        for it in range(max_iter + 1):
            a = zr * zr
            b = zi * zi
            s = a + b
            out = (s > bound) if test == 0 else ~(np.sqrt(s) < bound)
            live &= ~out
            if it == max_iter or not live.any():
                break
            t = zr * zi
            nzi = (t + t) + Ci
            nzr = (a - b) + Cr
            zr = np.where(live, nzr, zr)
            zi = np.where(live, nzi, zi)
            count += live.astype(np.uint32)
    return count


def fused_map(a, x, y):
    A, X, Y = (np.asarray(v, dtype=np.float32).astype(np.float64) for v in (a, x, y))
    kh, ke = np.float64(f32(-0.5)), np.float64(f32(1e-3))
    return (np.tanh(A * X + Y) * np.exp(kh * X * X) + np.sqrt(np.abs(Y) + ke)).astype(np.float32)


def row_softmax(m):
    M = np.asarray(m, dtype=np.float32).astype(np.float64)
    e = np.exp(M - M.max(axis=1, keepdims=True))
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


def mse_tanh(W, x, b, t, denom=None):
    """-> loss, dW, dx, db (all float64)."""
    W, x, b, t = (np.asarray(v, dtype=np.float32).astype(np.float64) for v in (W, x, b, t))
    denom = float(denom if denom else W.size)
    y = np.tanh(W * x + b[None, :])
    d = y - t
    loss = (d * d).sum() / denom
    g = 2.0 * d * (1.0 - y * y) / denom
    return loss, g * x, g * W, g.sum(axis=0)
