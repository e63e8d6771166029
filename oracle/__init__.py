"""CPU oracle for the data-parallel hot path -- TEST INFRASTRUCTURE, not product code.

Thin ctypes/numpy wrappers over ``libvernon_oracle.so`` (built from ``vernon_oracle.c`` by the
Makefile beside it).  Only the tests, the smoke check and the CPU-baseline leg of the benchmark
import this package; nothing under ``vernondsl_b200`` does.

Parity is UNPINNED by the reference: it holds no runnable implementation and no golden vector
for this path.  Loop semantics follow fractal.py:11-25 (test before update, count the updates,
square as (z0*z0 - z1*z1, (z1*z0)*2), coordinates at the pixel corner); every parameter comes
from the workload description.  ``numpy_restatement`` is a second, independently written
statement of the same rules used to cross-check the C code.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libvernon_oracle.so")

MANDELBROT, JULIA = 0, 1
TEST_NORM2_GT, TEST_NORM_GE = 0, 1
UNARY = {"tanh": 0, "exp": 1, "sqrt": 2, "abs": 3, "neg": 4, "square": 5, "recip": 6, "log": 7,
         "sigmoid": 8, "relu": 9, "cos": 10, "sin": 11, "rsqrt": 12}


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than its source."""
    src = os.path.join(_HERE, "vernon_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        fp = C.POINTER(C.c_float)
        dp = C.POINTER(C.c_double)
        up = C.POINTER(C.c_uint32)
        L.vo_num_threads.restype = C.c_int
        L.vo_set_num_threads.argtypes = [C.c_int]
        L.vo_escape_time.restype = C.c_uint64
        L.vo_escape_time.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_float, C.c_float,
                                     C.c_float, C.c_float, C.c_float, C.c_float, C.c_uint32,
                                     C.c_int, C.c_float, C.c_uint32, C.c_uint32, C.c_uint32, up]
        L.vo_escape_color.argtypes = [up, C.c_size_t, C.c_float, fp]
        L.vo_fused_map_f64.argtypes = [fp, fp, fp, C.c_size_t, fp, fp]
        L.vo_fused_map_bound.argtypes = [fp, fp, fp, C.c_size_t, C.c_double, dp]
        L.vo_unary_f64.argtypes = [C.c_int, fp, C.c_size_t, fp]
        L.vo_unary_f64.restype = C.c_int
        for name in ("vo_row_sum", "vo_row_max", "vo_row_softmax", "vo_col_sum"):
            getattr(L, name).argtypes = [fp, C.c_size_t, C.c_size_t, fp]
        L.vo_mse_tanh_fwd.restype = C.c_double
        L.vo_mse_tanh_fwd.argtypes = [fp, fp, fp, fp, C.c_size_t, C.c_size_t, C.c_double]
        L.vo_mse_tanh_bwd.argtypes = [fp, fp, fp, fp, C.c_size_t, C.c_size_t, C.c_double, fp, fp, dp]
        L.vo_digest_u32.argtypes = [up, C.c_size_t, C.c_uint64, C.POINTER(C.c_uint64),
                                    C.POINTER(C.c_uint64)]
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().vo_num_threads())


def set_num_threads(n: int) -> None:
    lib().vo_set_num_threads(int(n))


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def grid_steps(x0, x1, y0, y1, width, height):
    """Per-pixel steps, computed once in binary32 exactly as the host side of the library does:
    dx = (x1 - x0) / width, dy = (y1 - y0) / height (corner convention, fractal.py:20)."""
    f = np.float32
    dx = (f(x1) - f(x0)) / f(width)
    dy = (f(y1) - f(y0)) / f(height)
    return f(dx), f(dy)


def escape_time(kind, width, height, x0, y0, dx, dy, cr=0.0, ci=0.0, max_iter=256,
                test=TEST_NORM2_GT, bound=4.0, row_begin=0, row_step=1, row_count=None,
                want_image=True, fast=False):
    """Counts for rows row_begin, row_begin+row_step, ... -> (uint32 [row_count, width], sum).
    ``fast=True`` evaluates the contracted rounding sequence (see vo_escape_time_fast)."""
    if row_count is None:
        row_count = (height - row_begin + row_step - 1) // row_step
    out = np.empty((row_count, width), dtype=np.uint32) if want_image else None
    ptr = out.ctypes.data_as(C.POINTER(C.c_uint32)) if want_image else None
    if fast:
        if test != TEST_NORM2_GT:
            raise ValueError("the contracted mode only has the squared-norm test")
        fn = lib().vo_escape_time_fast
        fn.restype = C.c_uint64
        fn.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
                       C.c_float, C.c_uint32, C.c_float, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)]
        return out, int(fn(kind, width, height, x0, y0, dx, dy, cr, ci, max_iter, bound, row_begin, row_step,
                           row_count, ptr))
    total = lib().vo_escape_time(kind, width, height, x0, y0, dx, dy, cr, ci, max_iter, test,
                                 bound, row_begin, row_step, row_count, ptr)
    return out, int(total)


def escape_color(counts, scale):
    counts = np.ascontiguousarray(counts, dtype=np.uint32)
    out = np.empty(counts.shape, dtype=np.float32)
    lib().vo_escape_color(counts.ctypes.data_as(C.POINTER(C.c_uint32)), counts.size, scale,
                          out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def fused_map(a, x, y, want_scale=False):
    a, pa = _f32(a)
    x, px = _f32(x)
    y, py = _f32(y)
    out = np.empty(a.shape, dtype=np.float32)
    scale = np.empty(a.shape, dtype=np.float32) if want_scale else None
    lib().vo_fused_map_f64(pa, px, py, a.size, out.ctypes.data_as(C.POINTER(C.c_float)),
                           scale.ctypes.data_as(C.POINTER(C.c_float)) if want_scale else None)
    return (out, scale) if want_scale else out


def fused_map_bound(a, x, y, ulps=2.0):
    """Absolute error bound of the fused chain when each primitive map in it is within ``ulps`` ulp
    (first-order propagation, evaluated in binary64)."""
    a, pa = _f32(a)
    x, px = _f32(x)
    y, py = _f32(y)
    out = np.empty(a.shape, dtype=np.float64)
    lib().vo_fused_map_bound(pa, px, py, a.size, float(ulps), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def unary(op, x):
    x, px = _f32(x)
    out = np.empty(x.shape, dtype=np.float32)
    rc = lib().vo_unary_f64(UNARY[op], px, x.size, out.ctypes.data_as(C.POINTER(C.c_float)))
    if rc:
        raise ValueError(op)
    return out


def _rowop(name, m, out_shape):
    m, pm = _f32(m)
    rows, cols = m.shape
    out = np.empty(out_shape(rows, cols), dtype=np.float32)
    getattr(lib(), name)(pm, rows, cols, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def row_sum(m):
    return _rowop("vo_row_sum", m, lambda r, c: (r,))


def row_max(m):
    return _rowop("vo_row_max", m, lambda r, c: (r,))


def row_softmax(m):
    return _rowop("vo_row_softmax", m, lambda r, c: (r, c))


def col_sum(m):
    return _rowop("vo_col_sum", m, lambda r, c: (c,))


def mse_tanh_fwd(W, x, b, t, denom=None):
    W, pW = _f32(W)
    x, px = _f32(x)
    b, pb = _f32(b)
    t, pt = _f32(t)
    rows, cols = W.shape
    return float(lib().vo_mse_tanh_fwd(pW, px, pb, pt, rows, cols,
                                       float(denom if denom else rows * cols)))


def mse_tanh_bwd(W, x, b, t, denom=None):
    """-> (dW f32, dx f32, db f64) with g = 2*(y-t)*(1-y*y)/denom."""
    W, pW = _f32(W)
    x, px = _f32(x)
    b, pb = _f32(b)
    t, pt = _f32(t)
    rows, cols = W.shape
    dW = np.empty_like(W)
    dx = np.empty_like(W)
    db = np.empty(cols, dtype=np.float64)
    lib().vo_mse_tanh_bwd(pW, px, pb, pt, rows, cols, float(denom if denom else rows * cols),
                          dW.ctypes.data_as(C.POINTER(C.c_float)),
                          dx.ctypes.data_as(C.POINTER(C.c_float)),
                          db.ctypes.data_as(C.POINTER(C.c_double)))
    return dW, dx, db


def vertex_transform(pos, model, view, proj):
    """-> (gl_position [n,4], varying [n,3]); color.mlir:4-39 over an array of vertices, binary64."""
    pos, pp = _f32(pos)
    model, pm = _f32(model)
    view, pv = _f32(view)
    proj, pj = _f32(proj)
    n = pos.shape[0]
    out, var = np.empty((n, 4), dtype=np.float32), np.empty((n, 3), dtype=np.float32)
    fn = lib().vo_vertex_transform
    fn.argtypes = [C.POINTER(C.c_float)] * 4 + [C.c_size_t] + [C.POINTER(C.c_float)] * 2
    fn.restype = None
    fn(pp, pm, pv, pj, n, out.ctypes.data_as(C.POINTER(C.c_float)), var.ctypes.data_as(C.POINTER(C.c_float)))
    return out, var


def digest_u32(v, base_index=0):
    """(sum, position-weighted sum mod 2**64) of a uint32 array; exact integers."""
    v = np.ascontiguousarray(v, dtype=np.uint32)
    s, w = C.c_uint64(), C.c_uint64()
    lib().vo_digest_u32(v.ctypes.data_as(C.POINTER(C.c_uint32)), v.size, base_index,
                        C.byref(s), C.byref(w))
    return int(s.value), int(w.value)


def ulp_diff(got, want):
    """Distance in units of the last place of ``want`` (binary32), as float64 array."""
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    ulp = np.spacing(np.abs(want).astype(np.float32)).astype(np.float64)
    return np.abs(got.astype(np.float64) - want.astype(np.float64)) / ulp
