/*
 * vernon_oracle.c -- CPU restatement of the data-parallel hot path.  TEST INFRASTRUCTURE.
 *
 * This file is the checker the CUDA kernels are compared against, and the CPU baseline that
 * is timed beside them.  It is never linked into, loaded by or called from the shipped
 * library or package; only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * PARITY UNPINNED.  The reference project holds no implementation of this path that can run
 * here and no test, golden vector or fixture that pins a result: its only executable
 * statement of the path is the Taichi script fractal.py (third-party dependency taichi
 * 1.7.4, pinned in pyproject.toml:23 / uv.lock:504, not present, and driven through an
 * OpenGL ES backend, fractal.py:5).  What is followed here:
 *
 *   - loop semantics of the escape-time map: fractal.py:18-25 -- one independent evaluation
 *     per pixel, the escape test comes BEFORE the update, and the result counts the updates
 *     that were performed;
 *   - the complex square: fractal.py:11-13 -- (z0*z0 - z1*z1, (z1*z0)*2);
 *   - pixel coordinates from the integer index at the pixel CORNER: fractal.py:20;
 *   - every other operator (fused map chain, row sum / max / softmax, the tanh-MSE loss and
 *     its gradients) is defined by its formula only; those are evaluated in binary64 from
 *     the binary32 inputs and rounded once.
 *
 * Arithmetic contract of the exact escape-time mode (all binary32, round-to-nearest-even, no
 * fused multiply-add; compile with -ffp-contract=off):
 *
 *     x = x0 + (float)i * dx          y = y0 + (float)j * dy
 *     loop:  a = zr*zr;  b = zi*zi;  if (test(a+b)) stop;  if (it == max_iter) stop
 *            t = zr*zi;  zi = (t+t) + ci;  zr = (a-b) + cr;  ++it
 *
 * Build: see the Makefile beside this file.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define VO_EXPORT __attribute__((visibility("default")))

/* kinds */
enum { VO_MANDELBROT = 0, VO_JULIA = 1 };
/* escape tests */
enum { VO_TEST_NORM2_GT = 0, /* stop when a+b >  bound                          */
       VO_TEST_NORM_GE  = 1  /* stop when sqrtf(a+b) >= bound  (fractal.py:22)  */ };

VO_EXPORT int vo_version(void) { return 1; }

VO_EXPORT int vo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

VO_EXPORT void vo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* One pixel.  Follows fractal.py:21-24 (test first, then update, count the updates). */
static inline uint32_t escape_pixel(float zr, float zi, float cr, float ci, uint32_t max_iter,
                                    int test, float bound) {
  uint32_t it = 0;
  for (;;) {
    float a = zr * zr;
    float b = zi * zi;
    float s = a + b;
    int out = (test == VO_TEST_NORM2_GT) ? (s > bound) : !(sqrtf(s) < bound);
    if (out || it >= max_iter) break;
    float t = zr * zi;          /* fractal.py:13  z[1]*z[0]      */
    zi = (t + t) + ci;          /*                ... * 2 , + c  */
    zr = (a - b) + cr;          /* fractal.py:13  z0^2 - z1^2    */
    ++it;
  }
  return it;
}

/*
 * Escape-time map over selected rows of a width x height grid.
 * Rows visited: row_begin, row_begin+row_step, ... (row_count of them).  Row r of the visit
 * order is written to out + r*width (a compact [row_count][width] array).
 * kind = VO_MANDELBROT: z0 = 0, c = pixel.   kind = VO_JULIA: z0 = pixel, c = (cr, ci).
 * Returns the sum of all counts written.
 */
VO_EXPORT uint64_t vo_escape_time(int kind, uint32_t width, uint32_t height, float x0, float y0,
                                  float dx, float dy, float cr, float ci, uint32_t max_iter,
                                  int test, float bound, uint32_t row_begin, uint32_t row_step,
                                  uint32_t row_count, uint32_t *out) {
  uint64_t total = 0;
  (void)height;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : total)
  for (int64_t r = 0; r < (int64_t)row_count; ++r) {
    uint32_t j = row_begin + (uint32_t)r * row_step;
    float y = y0 + (float)j * dy;
    uint32_t *dst = out ? out + (size_t)r * width : NULL;
    uint64_t rowsum = 0;
    for (uint32_t i = 0; i < width; ++i) {
      float x = x0 + (float)i * dx;
      uint32_t it = (kind == VO_MANDELBROT)
                        ? escape_pixel(0.0f, 0.0f, x, y, max_iter, test, bound)
                        : escape_pixel(x, y, cr, ci, max_iter, test, bound);
      if (dst) dst[i] = it;
      rowsum += it;
    }
    total += rowsum;
  }
  return total;
}

/*
 * The contracted ("fast") arithmetic mode: the same loop with multiply-adds fused, as a compiler
 * with contraction enabled could emit it.  It is a different, but equally well-defined, rounding
 * sequence (fmaf is a single correctly rounded operation):
 *     test    s = fma(zi, zi, zr*zr)
 *     update  zi' = fma(zr+zr, zi, ci);   zr' = fma(zr, zr, fma(-zi, zi, cr))
 * Only the test "s > bound" exists in this mode.
 */
static inline uint32_t escape_pixel_fast(float zr, float zi, float cr, float ci, uint32_t max_iter,
                                         float bound) {
  uint32_t it = 0;
  for (;;) {
    float s = fmaf(zi, zi, zr * zr);
    if (!(s <= bound) || it >= max_iter) break;
    float nzi = fmaf(zr + zr, zi, ci);
    zr = fmaf(zr, zr, fmaf(-zi, zi, cr));
    zi = nzi;
    ++it;
  }
  return it;
}

VO_EXPORT uint64_t vo_escape_time_fast(int kind, uint32_t width, uint32_t height, float x0, float y0,
                                       float dx, float dy, float cr, float ci, uint32_t max_iter,
                                       float bound, uint32_t row_begin, uint32_t row_step,
                                       uint32_t row_count, uint32_t *out) {
  uint64_t total = 0;
  (void)height;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : total)
  for (int64_t r = 0; r < (int64_t)row_count; ++r) {
    uint32_t j = row_begin + (uint32_t)r * row_step;
    float y = y0 + (float)j * dy;
    uint32_t *dst = out ? out + (size_t)r * width : NULL;
    uint64_t rowsum = 0;
    for (uint32_t i = 0; i < width; ++i) {
      float x = x0 + (float)i * dx;
      uint32_t it = (kind == VO_MANDELBROT) ? escape_pixel_fast(0.0f, 0.0f, x, y, max_iter, bound)
                                            : escape_pixel_fast(x, y, cr, ci, max_iter, bound);
      if (dst) dst[i] = it;
      rowsum += it;
    }
    total += rowsum;
  }
  return total;
}

/* Colour written by fractal.py:25 from a count:  1 - iterations * scale  (binary32). */
VO_EXPORT void vo_escape_color(const uint32_t *counts, size_t n, float scale, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < (int64_t)n; ++k) out[k] = 1.0f - (float)counts[k] * scale;
}

/*
 * Fused map chain:  out = tanh(a*x + y) * exp(-0.5*x*x) + sqrt(|y| + 1e-3)
 * evaluated in binary64 from the binary32 inputs, rounded once.  The two constants are the
 * binary32 values the GPU graph holds (-0.5f, 1e-3f), promoted.
 * If `scale` is not NULL it receives, per element, the largest magnitude among the
 * intermediate values of the chain (used for the "2 ulp of the largest intermediate" bound).
 */
VO_EXPORT void vo_fused_map_f64(const float *a, const float *x, const float *y, size_t n,
                                float *out, float *scale) {
  const double kh = (double)-0.5f, ke = (double)1e-3f;
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < (int64_t)n; ++k) {
    double A = a[k], X = x[k], Y = y[k];
    double u = A * X + Y;
    double th = tanh(u);
    double e = exp(kh * X * X);
    double p = th * e;
    double q = sqrt(fabs(Y) + ke);
    double o = p + q;
    out[k] = (float)o;
    if (scale) {
      double m = fabs(u);
      if (fabs(A * X) > m) m = fabs(A * X);
      if (fabs(Y) > m) m = fabs(Y);
      if (fabs(th) > m) m = fabs(th);
      if (fabs(kh * X * X) > m) m = fabs(kh * X * X);
      if (e > m) m = e;
      if (fabs(p) > m) m = fabs(p);
      if (q > m) m = q;
      if (fabs(o) > m) m = fabs(o);
      scale[k] = (float)m;
    }
  }
}

static double ulp32(double v) {
  /* spacing of binary32 numbers at magnitude |v| (normal range) */
  int e;
  v = fabs(v);
  if (v < 1.17549435e-38) return 1.40129846e-45;
  frexp(v, &e);           /* v = m * 2^e, m in [0.5, 1) */
  return ldexp(1.0, e - 24);
}

/*
 * Forward error bound of the same chain when every primitive map in it (the fused multiply-add
 * a*x+y, tanh, the product x*x scaled by -0.5, exp, |y|+1e-3, sqrt, and the final fused
 * multiply-add) returns a value within `ulps` units in the last place of the correctly rounded
 * binary32 result for the inputs it was given.  First-order propagation:
 *     bound = ulps * sum over intermediates t of |d out / d t| * ulp32(t)
 * This is what "each map within N ulp" implies for the composite; an ulp of the final value
 * alone is not a usable unit because tanh(.)*exp(.) and sqrt(.) can cancel.
 */
VO_EXPORT void vo_fused_map_bound(const float *a, const float *x, const float *y, size_t n,
                                  double ulps, double *bound) {
  const double kh = (double)-0.5f, ke = (double)1e-3f;
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < (int64_t)n; ++k) {
    double A = a[k], X = x[k], Y = y[k];
    double u = A * X + Y, th = tanh(u), v = kh * X * X, e = exp(v);
    double w = fabs(Y) + ke, q = sqrt(w), o = th * e + q;
    double b = ulp32(u) * (1.0 - th * th) * e   /* u  -> tanh -> product */
             + ulp32(th) * e                    /* tanh result           */
             + ulp32(v) * e * fabs(th)          /* v  -> exp -> product  */
             + ulp32(e) * fabs(th)              /* exp result            */
             + ulp32(w) / (2.0 * q)             /* w  -> sqrt            */
             + ulp32(q)                         /* sqrt result           */
             + ulp32(o);                        /* final rounding        */
    bound[k] = ulps * b;
  }
}

/* Elementwise primitives in binary64, rounded once (for per-primitive ulp checks). */
enum { VO_U_TANH = 0, VO_U_EXP = 1, VO_U_SQRT = 2, VO_U_ABS = 3, VO_U_NEG = 4, VO_U_SQUARE = 5,
       VO_U_RECIP = 6, VO_U_LOG = 7, VO_U_SIGMOID = 8, VO_U_RELU = 9, VO_U_COS = 10,
       VO_U_SIN = 11, VO_U_RSQRT = 12 };

VO_EXPORT int vo_unary_f64(int op, const float *x, size_t n, float *out) {
  if (op < 0 || op > VO_U_RSQRT) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < (int64_t)n; ++k) {
    double v = x[k], r;
    switch (op) {
      case VO_U_TANH: r = tanh(v); break;
      case VO_U_EXP: r = exp(v); break;
      case VO_U_SQRT: r = sqrt(v); break;
      case VO_U_ABS: r = fabs(v); break;
      case VO_U_NEG: r = -v; break;
      case VO_U_SQUARE: r = v * v; break;
      case VO_U_RECIP: r = 1.0 / v; break;
      case VO_U_LOG: r = log(v); break;
      case VO_U_SIGMOID: r = 1.0 / (1.0 + exp(-v)); break;
      case VO_U_RELU: r = v > 0 ? v : 0; break;
      case VO_U_COS: r = cos(v); break;
      case VO_U_SIN: r = sin(v); break;
      default: r = 1.0 / sqrt(v); break;
    }
    out[k] = (float)r;
  }
  return 0;
}

/* Per-row sum and max of a row-major [rows][cols] matrix; binary64 accumulation. */
VO_EXPORT void vo_row_sum(const float *m, size_t rows, size_t cols, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const float *p = m + (size_t)r * cols;
    double s = 0.0;
    for (size_t c = 0; c < cols; ++c) s += p[c];
    out[r] = (float)s;
  }
}

VO_EXPORT void vo_row_max(const float *m, size_t rows, size_t cols, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const float *p = m + (size_t)r * cols;
    float mx = -INFINITY;
    for (size_t c = 0; c < cols; ++c) mx = p[c] > mx ? p[c] : mx;
    out[r] = mx;
  }
}

/* Numerically stable softmax along each row: exp(x - max) / sum exp(x - max), binary64. */
VO_EXPORT void vo_row_softmax(const float *m, size_t rows, size_t cols, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const float *p = m + (size_t)r * cols;
    float *o = out + (size_t)r * cols;
    double mx = -INFINITY;
    for (size_t c = 0; c < cols; ++c) mx = p[c] > mx ? p[c] : mx;
    double s = 0.0;
    for (size_t c = 0; c < cols; ++c) s += exp((double)p[c] - mx);
    for (size_t c = 0; c < cols; ++c) o[c] = (float)(exp((double)p[c] - mx) / s);
  }
}

/* Column sums of a row-major [rows][cols] matrix; binary64 accumulation. */
VO_EXPORT void vo_col_sum(const float *m, size_t rows, size_t cols, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < (int64_t)cols; ++c) {
    double s = 0.0;
    for (size_t r = 0; r < rows; ++r) s += m[r * cols + (size_t)c];
    out[c] = (float)s;
  }
}

/*
 * loss = mean over all [rows][cols] of (tanh(W*x + b[col]) - t)^2        (binary64)
 * `denom` is the element count the mean divides by (rows*cols of the WHOLE matrix, which is
 * larger than this call's rows*cols when the rows are one shard of several).
 * Returns the loss contribution of these rows, as a double.
 */
VO_EXPORT double vo_mse_tanh_fwd(const float *W, const float *x, const float *b, const float *t,
                                 size_t rows, size_t cols, double denom) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    double s = 0.0;
    for (size_t c = 0; c < cols; ++c) {
      size_t k = (size_t)r * cols + c;
      double y = tanh((double)W[k] * (double)x[k] + (double)b[c]);
      double d = y - (double)t[k];
      s += d * d;
    }
    total += s;
  }
  return total / denom;
}

/*
 * Gradients of the loss above:   g = 2*(y - t)*(1 - y*y)/denom,  y = tanh(W*x + b)
 *     dW = g*x     dx = g*W     db[col] = sum over rows of g                     (binary64)
 * db_acc (binary64, [cols]) receives the column sums unrounded; dW, dx are rounded once.
 */
VO_EXPORT void vo_mse_tanh_bwd(const float *W, const float *x, const float *b, const float *t,
                               size_t rows, size_t cols, double denom, float *dW, float *dx,
                               double *db_acc) {
  for (size_t c = 0; c < cols; ++c) db_acc[c] = 0.0;
#pragma omp parallel
  {
#ifdef _OPENMP
    int nth = omp_get_num_threads(), tid = omp_get_thread_num();
#else
    int nth = 1, tid = 0;
#endif
    /* each thread owns a contiguous range of columns: deterministic, no sharing */
    size_t c0 = cols * (size_t)tid / (size_t)nth, c1 = cols * (size_t)(tid + 1) / (size_t)nth;
    for (size_t r = 0; r < rows; ++r) {
      for (size_t c = c0; c < c1; ++c) {
        size_t k = r * cols + c;
        double y = tanh((double)W[k] * (double)x[k] + (double)b[c]);
        double g = 2.0 * (y - (double)t[k]) * (1.0 - y * y) / denom;
        dW[k] = (float)(g * (double)x[k]);
        dx[k] = (float)(g * (double)W[k]);
        db_acc[c] += g;
      }
    }
  }
}

/*
 * Vertex stage of the reference's shader input (source/tests/integration/color.mlir:4-39):
 * gl_position = proj * (view * (model * (p0, p1, p2, 1))) with row-major 4x4 matrices, varying = p.
 * Evaluated in binary64 from the binary32 inputs, rounded once.
 */
static void matvec4d(const float *M, const double *v, double *r) {
  for (int i = 0; i < 4; ++i)
    r[i] = (double)M[4 * i] * v[0] + (double)M[4 * i + 1] * v[1] + (double)M[4 * i + 2] * v[2] + (double)M[4 * i + 3] * v[3];
}

VO_EXPORT void vo_vertex_transform(const float *pos, const float *model, const float *view,
                                   const float *proj, size_t n, float *gl_position, float *varying) {
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < (int64_t)n; ++k) {
    double v[4] = {pos[3 * k], pos[3 * k + 1], pos[3 * k + 2], 1.0}, a[4], b[4], c[4];
    matvec4d(model, v, a);
    matvec4d(view, a, b);
    matvec4d(proj, b, c);
    for (int i = 0; i < 4; ++i) gl_position[4 * k + i] = (float)c[i];
    for (int i = 0; i < 3; ++i) varying[3 * k + i] = pos[3 * k + i];
  }
}

/*
 * Order-independent digest of a uint32 image: sum of counts, and a position-weighted
 * checksum  sum (k+1)*v[k]  mod 2^64.  Both are exact integer quantities, so a GPU image can
 * be compared with a stored oracle digest at sizes where the oracle takes minutes.
 */
VO_EXPORT void vo_digest_u32(const uint32_t *v, size_t n, uint64_t base_index, uint64_t *sum,
                             uint64_t *wsum) {
  uint64_t s = 0, w = 0;
#pragma omp parallel for schedule(static) reduction(+ : s, w)
  for (int64_t k = 0; k < (int64_t)n; ++k) {
    s += v[k];
    w += (base_index + (uint64_t)k + 1u) * (uint64_t)v[k];
  }
  *sum = s;
  *wsum = w;
}
