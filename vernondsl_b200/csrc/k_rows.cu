// Row reductions, softmax and column sums of a row-major [rows][cols] float matrix, sm_100a.
//
// HBM-bound.  Fast path (cols % 4 == 0 and cols <= 4096): ONE WARP PER ROW, the whole row held
// in registers (up to 32 float4 per lane), so the row is read from HBM exactly once even for
// softmax, every load of a row is in flight at once, and the reductions need warp shuffles only
// (no shared memory, no block barrier).  Any other shape takes a block-per-row kernel that
// re-reads the row through L1/L2.  Summation order is fixed, so results are bit-reproducible.
// The reference project has no counterpart for these operators.
#include <cfloat>
#include <cstring>

#include "vrhi_internal.h"

namespace vrhi {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

enum { ROW_SUM = 1, ROW_MAX = 2, ROW_SOFTMAX = 4 };

// NV = float4 groups per lane (row length <= NV*128 floats).  WHAT = bit set of outputs.
template <int NV, int WHAT>
__global__ void __launch_bounds__(256) row_warp_kernel(const float4 *__restrict__ in, float *__restrict__ out_sum,
                                                       float *__restrict__ out_max, float4 *__restrict__ out_soft,
                                                       uint64_t rows, uint32_t cols4) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t n_warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = warp; r < rows; r += n_warps) {
    const float4 *src = in + r * cols4;
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t c = lane + 32u * k;
      // lanes past the row end hold the identity of both reductions' inputs
      v[k] = (c < cols4) ? __ldcs(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.f, m = -FLT_MAX;
    if (WHAT & ROW_SUM) {
#pragma unroll
      for (int k = 0; k < NV; ++k) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
      s = warp_sum(s);
    }
    if (WHAT & (ROW_MAX | ROW_SOFTMAX)) {
      float mm = -INFINITY;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t c = lane + 32u * k;
        if (c < cols4) mm = fmaxf(mm, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
      }
      m = warp_max(mm);
    }
    if (lane == 0) {
      if (WHAT & ROW_SUM) out_sum[r] = s;
      if (WHAT & ROW_MAX) out_max[r] = m;
    }
    if (WHAT & ROW_SOFTMAX) {
      float z = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t c = lane + 32u * k;
        if (c < cols4) {
          v[k].x = expf(v[k].x - m); v[k].y = expf(v[k].y - m);
          v[k].z = expf(v[k].z - m); v[k].w = expf(v[k].w - m);
          z += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
      }
      z = warp_sum(z);
      const float inv = 1.0f / z;
      float4 *dst = out_soft + r * cols4;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t c = lane + 32u * k;
        if (c < cols4) __stcs(dst + c, make_float4(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv));
      }
    }
  }
}

// exp(x - m) as 2^(x*log2e - m*log2e): one fused multiply-add and one MUFU.EX2 per element.
// ml = m*log2e is rounded once per row; that rounding is a common factor of every element of the
// row and cancels in the normalisation.  Relative error per element stays below 2e-6 for
// |x - m| < 60 (fma rounding of the exponent plus the 2^-22 of ex2.approx).
__device__ __forceinline__ float exp2_approx(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}

// Softmax rows: WPR warps share one row (8 float4 per thread at most), so a 256-thread CTA works
// on 8/WPR rows at a time with ~64 registers per thread and 32 resident warps per SM: enough
// independent warps to keep loads in flight while others are in their exp phase.  The row still
// makes exactly one trip from HBM and one back.  Cross-warp reductions go through three separate
// shared arrays (sum, max, normaliser), one CTA barrier each; partials are combined in warp
// order, so results do not depend on scheduling.
template <int NV, int WPR, int WHAT>
__global__ void __launch_bounds__(256) row_group_kernel(const float4 *__restrict__ in, float *__restrict__ out_sum,
                                                        float *__restrict__ out_max, float4 *__restrict__ out_soft,
                                                        uint64_t rows, uint32_t cols4) {
  constexpr int GROUPS = 8 / WPR;
  constexpr uint32_t TPR = 32u * WPR;  // threads per row
  __shared__ float red_sum[8], red_max[8], red_z[8];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t group = warp / WPR, wig = warp % WPR;
  const uint32_t t = wig * 32u + lane;
  const float kLog2e = 1.4426950408889634f;
  for (uint64_t base = (uint64_t)blockIdx.x * GROUPS; base < rows; base += (uint64_t)gridDim.x * GROUPS) {
    const uint64_t r = base + group;
    const bool active = r < rows;
    const float4 *src = in + r * cols4;
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t c = t + TPR * k;
      v[k] = (active && c < cols4) ? __ldcs(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.f, mm = -INFINITY;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const uint32_t c = t + TPR * k;
      if (WHAT & ROW_SUM) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
      if (c < cols4) mm = fmaxf(mm, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
    }
    if (WHAT & ROW_SUM) s = warp_sum(s);
    mm = warp_max(mm);
    if (WPR > 1) {
      if (lane == 0) {
        if (WHAT & ROW_SUM) red_sum[warp] = s;
        red_max[warp] = mm;
      }
      __syncthreads();
      s = 0.f; mm = -INFINITY;
#pragma unroll
      for (int j = 0; j < WPR; ++j) {
        if (WHAT & ROW_SUM) s += red_sum[group * WPR + j];
        mm = fmaxf(mm, red_max[group * WPR + j]);
      }
    }
    if (active && t == 0) {
      if (WHAT & ROW_SUM) out_sum[r] = s;
      if (WHAT & ROW_MAX) out_max[r] = mm;
    }
    if (WHAT & ROW_SOFTMAX) {
      const float ml = -mm * kLog2e;
      float z = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t c = t + TPR * k;
        if (c < cols4) {
          v[k].x = exp2_approx(fmaf(v[k].x, kLog2e, ml)); v[k].y = exp2_approx(fmaf(v[k].y, kLog2e, ml));
          v[k].z = exp2_approx(fmaf(v[k].z, kLog2e, ml)); v[k].w = exp2_approx(fmaf(v[k].w, kLog2e, ml));
          z += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
      }
      z = warp_sum(z);
      if (WPR > 1) {
        if (lane == 0) red_z[warp] = z;
        __syncthreads();
        z = 0.f;
#pragma unroll
        for (int j = 0; j < WPR; ++j) z += red_z[group * WPR + j];
      }
      const float inv = 1.0f / z;
      float4 *dst = out_soft + r * cols4;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const uint32_t c = t + TPR * k;
        if (active && c < cols4) __stcs(dst + c, make_float4(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv));
      }
    }
  }
}

// Any shape: one 256-thread block per row, scalar accesses, three passes for softmax.
__device__ __forceinline__ float block_reduce(float v, bool is_max, float *smem) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();  // smem reuse across consecutive calls
  if (l == 0) smem[w] = v;
  __syncthreads();
  float r = (l < 8) ? smem[l] : (is_max ? -INFINITY : 0.f);
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

template <int WHAT>
__global__ void __launch_bounds__(256) row_block_kernel(const float *__restrict__ in, float *__restrict__ out_sum,
                                                        float *__restrict__ out_max, float *__restrict__ out_soft,
                                                        uint64_t rows, uint64_t cols) {
  __shared__ float smem[8];
  for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float *src = in + r * cols;
    float s = 0.f, m = -INFINITY;
    for (uint64_t c = threadIdx.x; c < cols; c += 256) {
      float x = src[c];
      s += x;
      m = fmaxf(m, x);
    }
    if (WHAT & ROW_SUM) {
      s = block_reduce(s, false, smem);
      if (threadIdx.x == 0) out_sum[r] = s;
    }
    if (WHAT & (ROW_MAX | ROW_SOFTMAX)) {
      m = block_reduce(m, true, smem);
      if ((WHAT & ROW_MAX) && threadIdx.x == 0) out_max[r] = m;
    }
    if (WHAT & ROW_SOFTMAX) {
      float z = 0.f;
      for (uint64_t c = threadIdx.x; c < cols; c += 256) z += expf(src[c] - m);
      z = block_reduce(z, false, smem);
      const float inv = 1.0f / z;
      float *dst = out_soft + r * cols;
      for (uint64_t c = threadIdx.x; c < cols; c += 256) dst[c] = expf(src[c] - m) * inv;
    }
  }
}

template <int WHAT>
static int launch_rows(vrhi_stream_t *st, const float *in, float *osum, float *omax, float *osoft, uint64_t rows, uint64_t cols,
                       const char *name) {
  const int sms = st->dev->prop.multiProcessorCount;
  if ((WHAT & ROW_SOFTMAX) && cols % 4 == 0 && cols <= 8192) {
    const uint32_t cols4 = (uint32_t)(cols / 4);
    const float4 *i4 = (const float4 *)in;
    float4 *o4 = (float4 *)osoft;
    const int wpr = cols4 <= 256 ? 1 : cols4 <= 512 ? 2 : cols4 <= 1024 ? 4 : 8;
    const uint32_t nv = (cols4 + 32u * wpr - 1) / (32u * wpr);
    const uint64_t groups = 8 / wpr;
    uint64_t want = (rows + groups - 1) / groups;
    // one CTA per group of rows, not a persistent grid: measured on B200, letting the hardware
    // scheduler stream CTAs (each loads, reduces, writes and leaves) beats a resident grid whose
    // CTAs fall into lock step, all loading and then all storing (0.314 ms against 0.36 ms on [65536,4096])
    uint64_t cap = 0x7fffffffull;
    unsigned grid = (unsigned)(want < cap ? want : cap);
#define GROUP_LAUNCH(NV, WPR) row_group_kernel<NV, WPR, (WHAT | ROW_SOFTMAX)><<<grid, 256, 0, st->s>>>(i4, osum, omax, o4, rows, cols4)
#define GROUP_NV(WPR)                 \
  do {                                \
    if (nv <= 1) GROUP_LAUNCH(1, WPR); \
    else if (nv <= 2) GROUP_LAUNCH(2, WPR); \
    else if (nv <= 4) GROUP_LAUNCH(4, WPR); \
    else GROUP_LAUNCH(8, WPR);        \
  } while (0)
    if (wpr == 1) GROUP_NV(1);
    else if (wpr == 2) GROUP_NV(2);
    else if (wpr == 4) GROUP_NV(4);
    else GROUP_NV(8);
#undef GROUP_NV
#undef GROUP_LAUNCH
  } else if (cols % 4 == 0 && cols <= 4096) {
    const uint32_t cols4 = (uint32_t)(cols / 4);
    const uint32_t nv = (cols4 + 31) / 32;
    // softmax keeps the row live across two reductions: fewer resident warps, so more CTAs of
    // rows in flight do not help; 8 warps per CTA, CTAs = min(rows/8, SMs * 8)
    uint64_t want = (rows + 7) / 8;
    uint64_t cap = (uint64_t)sms * 8;
    unsigned grid = (unsigned)(want < cap ? want : cap);
    const float4 *i4 = (const float4 *)in;
    float4 *o4 = (float4 *)osoft;
#define ROWS_LAUNCH(NV) row_warp_kernel<NV, WHAT><<<grid, 256, 0, st->s>>>(i4, osum, omax, o4, rows, cols4)
    if (nv <= 1) ROWS_LAUNCH(1);
    else if (nv <= 2) ROWS_LAUNCH(2);
    else if (nv <= 4) ROWS_LAUNCH(4);
    else if (nv <= 8) ROWS_LAUNCH(8);
    else if (nv <= 16) ROWS_LAUNCH(16);
    else ROWS_LAUNCH(32);
#undef ROWS_LAUNCH
  } else {
    uint64_t cap = (uint64_t)sms * 8;
    unsigned grid = (unsigned)(rows < cap ? rows : cap);
    row_block_kernel<WHAT><<<grid, 256, 0, st->s>>>(in, osum, omax, osoft, rows, cols);
  }
  return post_launch(st, name);
}

static int rows_common(const ArgView *args, int n_args, int want_args, const void *params, size_t params_size,
                       vrhi_rows_params *q, const char *name) {
  VRHI_TRY(read_params(params, params_size, q));
  if (n_args != want_args) return fail(VRHI_ERR_INVALID, "%s takes %d arguments, got %d", name, want_args, n_args);
  if (q->cols == 0 && q->rows != 0) return fail(VRHI_ERR_SIZE, "%s: rows of zero length", name);
  if (q->rows > (1ull << 40) || q->cols > (1ull << 32)) return fail(VRHI_ERR_SIZE, "%s: shape out of range", name);
  uint64_t elements = 0;
  VRHI_TRY(element_count(q->rows, q->cols, name, &elements));
  if (args[0].bytes < elements * 4) return fail(VRHI_ERR_SIZE, "%s: input holds %llu bytes, %llu needed", name, (unsigned long long)args[0].bytes, (unsigned long long)(q->rows * q->cols * 4));
  for (int k = 1; k < n_args; ++k)
    if (!writable(args[k])) return fail(VRHI_ERR_INVALID, "%s: argument %d is read-only (class %s)", name, k, vrhi_arg_class_name(args[k].buf_cls));
  return VRHI_OK;
}

static int need(const ArgView &a, uint64_t bytes, const char *name, int k) {
  if (a.bytes < bytes) return fail(VRHI_ERR_SIZE, "%s: argument %d holds %llu bytes, %llu needed", name, k, (unsigned long long)a.bytes, (unsigned long long)bytes);
  return VRHI_OK;
}

int launch_row_sum(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_rows_params q;
  VRHI_TRY(rows_common(args, n_args, 2, params, params_size, &q, "row_sum"));
  if (q.rows == 0) return VRHI_OK;
  VRHI_TRY(need(args[1], q.rows * 4, "row_sum", 1));
  return launch_rows<ROW_SUM>(st, (const float *)args[0].ptr, (float *)args[1].ptr, nullptr, nullptr, q.rows, q.cols, "row_sum");
}

int launch_row_max(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_rows_params q;
  VRHI_TRY(rows_common(args, n_args, 2, params, params_size, &q, "row_max"));
  if (q.rows == 0) return VRHI_OK;
  VRHI_TRY(need(args[1], q.rows * 4, "row_max", 1));
  return launch_rows<ROW_MAX>(st, (const float *)args[0].ptr, nullptr, (float *)args[1].ptr, nullptr, q.rows, q.cols, "row_max");
}

int launch_row_softmax(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_rows_params q;
  VRHI_TRY(rows_common(args, n_args, 2, params, params_size, &q, "row_softmax"));
  if (q.rows == 0) return VRHI_OK;
  VRHI_TRY(need(args[1], q.rows * q.cols * 4, "row_softmax", 1));
  return launch_rows<ROW_SOFTMAX>(st, (const float *)args[0].ptr, nullptr, nullptr, (float *)args[1].ptr, q.rows, q.cols, "row_softmax");
}

int launch_row_stats_softmax(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_rows_params q;
  VRHI_TRY(rows_common(args, n_args, 4, params, params_size, &q, "row_stats_softmax"));
  if (q.rows == 0) return VRHI_OK;
  VRHI_TRY(need(args[1], q.rows * 4, "row_stats_softmax", 1));
  VRHI_TRY(need(args[2], q.rows * 4, "row_stats_softmax", 2));
  VRHI_TRY(need(args[3], q.rows * q.cols * 4, "row_stats_softmax", 3));
  return launch_rows<ROW_SUM | ROW_MAX | ROW_SOFTMAX>(st, (const float *)args[0].ptr, (float *)args[1].ptr, (float *)args[2].ptr,
                                                       (float *)args[3].ptr, q.rows, q.cols, "row_stats_softmax");
}

// ---------------------------------------------------------------------------------------------
// Column sums.  Stage 1: a thread owns four adjacent columns and walks down a fixed set of rows
// (grid.y row groups), writing one partial row per group.  Stage 2 adds the partial rows in
// index order.  No atomics: the result does not depend on scheduling.
__global__ void __launch_bounds__(256) col_partial_kernel(const float *__restrict__ in, float *__restrict__ partial,
                                                          uint64_t rows, uint64_t cols) {
  const uint64_t c0 = ((uint64_t)blockIdx.x * 256 + threadIdx.x) * 4;
  if (c0 >= cols) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if ((cols & 3u) == 0) {
    const float4 *p = reinterpret_cast<const float4 *>(in + c0);
    const uint64_t cols4 = cols / 4;
    for (uint64_t r = blockIdx.y; r < rows; r += gridDim.y) {
      float4 v = __ldcs(p + r * cols4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  } else {
    for (uint64_t r = blockIdx.y; r < rows; r += gridDim.y) {
      const float *p = in + r * cols + c0;
      acc.x += p[0];
      if (c0 + 1 < cols) acc.y += p[1];
      if (c0 + 2 < cols) acc.z += p[2];
      if (c0 + 3 < cols) acc.w += p[3];
    }
  }
  float *dst = partial + (uint64_t)blockIdx.y * cols + c0;
  dst[0] = acc.x;
  if (c0 + 1 < cols) dst[1] = acc.y;
  if (c0 + 2 < cols) dst[2] = acc.z;
  if (c0 + 3 < cols) dst[3] = acc.w;
}

__global__ void __launch_bounds__(256) col_finalize_kernel(const float *__restrict__ partial, float *__restrict__ out,
                                                           uint32_t groups, uint64_t cols, float scale) {
  // A block owns 32 adjacent columns; its eight warps each add every eighth partial row (so the
  // loads of one warp are coalesced and independent), and the eight slice sums are combined in a
  // fixed tree.  The result depends on `groups` only, never on scheduling.
  __shared__ float sm[8][33];
  const uint32_t lane = threadIdx.x & 31u, slice = threadIdx.x >> 5;
  const uint64_t c = (uint64_t)blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < cols)
    for (uint32_t g = slice; g < groups; g += 8) s += partial[(uint64_t)g * cols + c];
  sm[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && c < cols)
    out[c] = (((sm[0][lane] + sm[1][lane]) + (sm[2][lane] + sm[3][lane])) + ((sm[4][lane] + sm[5][lane]) + (sm[6][lane] + sm[7][lane]))) * scale;
}

// Shared with the backward kernel: sums `groups` partial rows of `cols` floats into out.
int col_finalize(vrhi_stream_t *st, const float *partial, float *out, uint32_t groups, uint64_t cols, float scale) {
  col_finalize_kernel<<<(unsigned)((cols + 31) / 32), 256, 0, st->s>>>(partial, out, groups, cols, scale);
  return post_launch(st, "col_finalize");
}

int launch_col_sum(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_rows_params q;
  VRHI_TRY(rows_common(args, n_args, 2, params, params_size, &q, "col_sum"));
  if (q.cols == 0) return VRHI_OK;
  VRHI_TRY(need(args[1], q.cols * 4, "col_sum", 1));
  if (q.rows == 0) {
    VRHI_CUDA(cudaMemsetAsync(args[1].ptr, 0, q.cols * 4, st->s));
    return VRHI_OK;
  }
  const int sms = st->dev->prop.multiProcessorCount;
  const uint64_t gx = (q.cols + 1023) / 1024;
  uint64_t gy = ((uint64_t)sms * 8 + gx - 1) / gx;
  if (gy > q.rows) gy = q.rows;
  if (gy > 1024) gy = 1024;
  char *payload = nullptr;
  VRHI_TRY(stream_arena(st, gy * q.cols * 4, nullptr, &payload));
  dim3 grid((unsigned)gx, (unsigned)gy);
  col_partial_kernel<<<grid, 256, 0, st->s>>>((const float *)args[0].ptr, (float *)payload, q.rows, q.cols);
  VRHI_TRY(post_launch(st, "col_sum"));
  return col_finalize(st, (const float *)payload, (float *)args[1].ptr, (uint32_t)gy, q.cols, 1.0f);
}

}  // namespace vrhi

// ---------------------------------------------------------------------------------------------
// Column sums for callers that must not allocate.
//
// Some users of this library sit where an allocation is not an option: a frame or control loop
// with a hard latency budget (cudaMalloc can take milliseconds and serialises the device), a
// process whose HBM was carved up front between tenants so that nothing may grow later, or code
// running between other people's kernels that may not disturb the allocator's state.  Every
// other operator here takes its scratch from a per-stream arena that is allocated on first use
// and may grow; this entry point instead keeps the per-row-group partial sums in a fixed array
// that is part of the library image.  Cost: each GPU that loads the library holds the array
// (kStaticPartialFloats * 4 bytes = 1 MiB) until the process exits.
//
// Use: the first call on a device asks CUDA for the array's device address (a lookup, not an
// allocation); let that first call happen before any stream capture is begun.  The array is
// shared by every call on the device and keeps whatever the last call left in it, so two calls
// whose kernels could run at the same time (different streams with no ordering between them)
// race; calls on one stream, or ordered by events, are safe.  No call here reaches cudaMalloc,
// cudaFree or any allocating library routine.
#include <mutex>

namespace {

constexpr uint64_t kStaticPartialFloats = 262144;  // 1 MiB: e.g. 64 row groups of 4096 columns
static __device__ __align__(256) float g_static_col_partials[kStaticPartialFloats];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float *g_static_partials_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal
int g_static_sm_count[kMaxDevices] = {};

// The array's name is only a host-side stand-in: the device address has to be asked for, once
// per device, with that device current.
int static_scratch_for_current_device(float **out_ptr, int *out_sms) {
  int dev = -1;
  VRHI_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return vrhi::fail(VRHI_ERR_UNSUPPORTED, "device ordinal %d is beyond the %d this entry point tracks", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_partials_ptr[dev]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_col_partials);
    if (e != cudaSuccess || !p) return vrhi::fail(VRHI_ERR_CUDA, "cudaGetSymbolAddress(static column partials) failed: %s", cudaGetErrorString(e));
    int sms = 0;
    VRHI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_static_sm_count[dev] = sms;
    g_static_partials_ptr[dev] = static_cast<float *>(p);
  }
  *out_ptr = g_static_partials_ptr[dev];
  *out_sms = g_static_sm_count[dev];
  return VRHI_OK;
}

}  // namespace

extern "C" int vrhi_col_sum_static_scratch(const float *in_device, float *out_device, uint64_t rows, uint64_t cols,
                                           void *cuda_stream) {
  using namespace vrhi;
  if (!in_device || !out_device) return fail(VRHI_ERR_INVALID, "col_sum_static_scratch: NULL pointer");
  if (cols == 0) return VRHI_OK;
  if (cols > kStaticPartialFloats)
    return fail(VRHI_ERR_SIZE, "col_sum_static_scratch: %llu columns exceed the fixed scratch (%llu floats); use the col_sum operator", (unsigned long long)cols, (unsigned long long)kStaticPartialFloats);
  if (rows > (1ull << 40)) return fail(VRHI_ERR_SIZE, "col_sum_static_scratch: row count out of range");
  if (reinterpret_cast<uintptr_t>(in_device) % 16 || reinterpret_cast<uintptr_t>(out_device) % 4)
    return fail(VRHI_ERR_SIZE, "col_sum_static_scratch: input must be 16-byte aligned and output 4-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  if (rows == 0) {
    VRHI_CUDA(cudaMemsetAsync(out_device, 0, cols * 4, s));
    return VRHI_OK;
  }
  float *partials = nullptr;
  int sms = 0;
  VRHI_TRY(static_scratch_for_current_device(&partials, &sms));
  const uint64_t gx = (cols + 1023) / 1024;
  uint64_t gy = ((uint64_t)sms * 8 + gx - 1) / gx;
  if (gy > rows) gy = rows;
  if (gy > 1024) gy = 1024;
  if (gy > kStaticPartialFloats / cols) gy = kStaticPartialFloats / cols;  // >= 1 by the check above
  // Stage 1 writes every partial that stage 2 reads (gy rows of `cols` floats), so nothing in the
  // array has to be cleared and whatever an earlier call left behind is never read.
  dim3 grid((unsigned)gx, (unsigned)gy);
  col_partial_kernel<<<grid, 256, 0, s>>>(in_device, partials, rows, cols);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(VRHI_ERR_CUDA, "launch of col_sum_static_scratch (partials) failed: %s", cudaGetErrorString(e));
  col_finalize_kernel<<<(unsigned)((cols + 31) / 32), 256, 0, s>>>(partials, out_device, (uint32_t)gy, cols, 1.0f);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(VRHI_ERR_CUDA, "launch of col_sum_static_scratch (finalize) failed: %s", cudaGetErrorString(e));
  return VRHI_OK;
}
