// Per-element shader-style maps: the arithmetic of the reference's shader input file
// (source/tests/integration/color.mlir) as plain CUDA kernels over arrays.
//
//   vertex stage (color.mlir:4-39): extend each position (p0,p1,p2) to (p0,p1,p2,1), apply the
//     model, view and projection matrices one after the other (the three linalg.matvec steps the
//     file sketches at :29-36), emit gl_Position and pass the position through as the varying;
//   fragment stage (color.mlir:43-59): extend the uniform colour (c0,c1,c2) to (c0,c1,c2,1) for
//     every fragment of a pixel buffer.
//
// No graphics API is involved: inputs and outputs are device arrays, the "pixel buffer" is a
// headless [n][4] float array.  Both kernels are HBM-bound (28 + 12 bytes per vertex, 16 bytes per
// fragment).  Each matrix row is applied as one multiply and three fused multiply-adds, left to
// right.
#include <cstring>

#include "vrhi_internal.h"

namespace vrhi {

struct Mat4 {
  float m[16];  // row-major
};

__device__ __forceinline__ float4 matvec4(const Mat4 &M, float4 v) {
  float4 r;
  r.x = fmaf(M.m[3], v.w, fmaf(M.m[2], v.z, fmaf(M.m[1], v.y, M.m[0] * v.x)));
  r.y = fmaf(M.m[7], v.w, fmaf(M.m[6], v.z, fmaf(M.m[5], v.y, M.m[4] * v.x)));
  r.z = fmaf(M.m[11], v.w, fmaf(M.m[10], v.z, fmaf(M.m[9], v.y, M.m[8] * v.x)));
  r.w = fmaf(M.m[15], v.w, fmaf(M.m[14], v.z, fmaf(M.m[13], v.y, M.m[12] * v.x)));
  return r;
}

__global__ void __launch_bounds__(256) vertex_transform_kernel(const float *__restrict__ pos, const float *__restrict__ model,
                                                               const float *__restrict__ view, const float *__restrict__ proj,
                                                               float4 *__restrict__ out_pos, float *__restrict__ out_varying,
                                                               uint64_t n) {
  __shared__ Mat4 sm[3];
  if (threadIdx.x < 48) {
    const float *src = threadIdx.x < 16 ? model : (threadIdx.x < 32 ? view : proj);
    sm[threadIdx.x / 16].m[threadIdx.x % 16] = src[threadIdx.x % 16];
  }
  __syncthreads();
  const Mat4 Mm = sm[0], Mv = sm[1], Mp = sm[2];
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t k = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) {
    const float p0 = pos[3 * k], p1 = pos[3 * k + 1], p2 = pos[3 * k + 2];
    float4 v = make_float4(p0, p1, p2, 1.0f);
    v = matvec4(Mm, v);
    v = matvec4(Mv, v);
    v = matvec4(Mp, v);
    __stcs(out_pos + k, v);
    out_varying[3 * k] = p0;
    out_varying[3 * k + 1] = p1;
    out_varying[3 * k + 2] = p2;
  }
}

__global__ void __launch_bounds__(256) flat_color_kernel(const float *__restrict__ color, float4 *__restrict__ out, uint64_t n) {
  const float4 c = make_float4(color[0], color[1], color[2], 1.0f);
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t k = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) __stcs(out + k, c);
}

static unsigned grid_for(vrhi_stream_t *st, uint64_t n) {
  const uint64_t cap = (uint64_t)st->dev->prop.multiProcessorCount * 8;
  uint64_t want = (n + 255) / 256;
  return (unsigned)(want < cap ? (want ? want : 1) : cap);
}

int launch_vertex_transform(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_map_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 6) return fail(VRHI_ERR_INVALID, "vertex_transform takes 6 arguments (pos, model, view, proj, gl_position, varying), got %d", n_args);
  if (q.n == 0) return VRHI_OK;
  const uint64_t need[6] = {q.n * 12, 64, 64, 64, q.n * 16, q.n * 12};
  for (int k = 0; k < 6; ++k)
    if (args[k].bytes < need[k]) return fail(VRHI_ERR_SIZE, "vertex_transform: argument %d holds %llu bytes, %llu needed", k, (unsigned long long)args[k].bytes, (unsigned long long)need[k]);
  if (!writable(args[4]) || !writable(args[5])) return fail(VRHI_ERR_INVALID, "vertex_transform: an output buffer is read-only");
  vertex_transform_kernel<<<grid_for(st, q.n), 256, 0, st->s>>>((const float *)args[0].ptr, (const float *)args[1].ptr, (const float *)args[2].ptr,
                                                                (const float *)args[3].ptr, (float4 *)args[4].ptr, (float *)args[5].ptr, q.n);
  return post_launch(st, "vertex_transform");
}

int launch_flat_color(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_map_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 2) return fail(VRHI_ERR_INVALID, "flat_color takes 2 arguments (color, fragments), got %d", n_args);
  if (q.n == 0) return VRHI_OK;
  if (args[0].bytes < 12) return fail(VRHI_ERR_SIZE, "flat_color: the colour needs 12 bytes");
  if (args[1].bytes < q.n * 16) return fail(VRHI_ERR_SIZE, "flat_color: the fragment buffer holds %llu bytes, %llu needed", (unsigned long long)args[1].bytes, (unsigned long long)q.n * 16);
  if (!writable(args[1])) return fail(VRHI_ERR_INVALID, "flat_color: the fragment buffer is read-only");
  flat_color_kernel<<<grid_for(st, q.n), 256, 0, st->s>>>((const float *)args[0].ptr, (float4 *)args[1].ptr, q.n);
  return post_launch(st, "flat_color");
}

}  // namespace vrhi
