// Per-element map kernels, sm_100a: the specialised fused chain of the map workload, and a
// generic fused-tape kernel that runs any chain of elementwise operations in one pass.
//
// Both are HBM-bound by design: 128-bit streaming loads and stores, grid sized to a multiple of
// the SM count, several independent loads in flight per thread.  The reference project has no
// counterpart; the chain's formula is the workload definition
//     out = tanh(a*x + y) * exp(-0.5*x*x) + sqrt(|y| + 1e-3).
#include <cstring>

#include "tape_math.cuh"
#include "vrhi_internal.h"

namespace vrhi {

__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { __stcs(p, v); }

__device__ __forceinline__ float chain_one(float a, float x, float y) {
  float u = fmaf(a, x, y);
  float th = tanhf(u);
  // exp(-x*x/2): the product is rounded once (hx = -x/2 is exact), and its rounding error vl,
  // recovered exactly by the fma, is folded back in as exp(vh + vl) = exp(vh) * (1 + vl)
  const float hx = -0.5f * x;
  const float vh = hx * x;
  const float vl = fmaf(hx, x, -vh);
  float e = expf(vh);
  e = fmaf(e, vl, e);
  float q = sqrtf(fabsf(y) + 1e-3f);
  return fmaf(th, e, q);
}

__device__ __forceinline__ float4 chain_four(float4 a, float4 x, float4 y) {
  return make_float4(chain_one(a.x, x.x, y.x), chain_one(a.y, x.y, y.y), chain_one(a.z, x.z, y.z),
                     chain_one(a.w, x.w, y.w));
}

// Each thread owns UNROLL float4 groups per trip, strided by the grid so that every warp's
// accesses stay contiguous.
template <int UNROLL>
__global__ void __launch_bounds__(256) fused_map_kernel(const float4 *__restrict__ a, const float4 *__restrict__ x,
                                                        const float4 *__restrict__ y, float4 *__restrict__ out,
                                                        uint64_t n4, uint64_t n, const float *a1, const float *x1,
                                                        const float *y1, float *o1) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  uint64_t k = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; k + (UNROLL - 1) * stride < n4; k += UNROLL * stride) {
    float4 va[UNROLL], vx[UNROLL], vy[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      va[u] = ld_stream(a + k + u * stride);
      vx[u] = ld_stream(x + k + u * stride);
      vy[u] = ld_stream(y + k + u * stride);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) st_stream(out + k + u * stride, chain_four(va[u], vx[u], vy[u]));
  }
  for (; k < n4; k += stride) st_stream(out + k, chain_four(ld_stream(a + k), ld_stream(x + k), ld_stream(y + k)));
  // ragged tail (n not a multiple of 4): at most 3 elements, first block only
  if (blockIdx.x == 0 && threadIdx.x < (n & 3u)) {
    uint64_t e = n4 * 4 + threadIdx.x;
    o1[e] = chain_one(a1[e], x1[e], y1[e]);
  }
}

int launch_fused_map(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_map_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 4) return fail(VRHI_ERR_INVALID, "fused_map takes 4 arguments (a, x, y, out), got %d", n_args);
  if (q.n == 0) return VRHI_OK;
  for (int k = 0; k < 4; ++k)
    if (args[k].bytes < q.n * 4) return fail(VRHI_ERR_SIZE, "fused_map: argument %d holds %llu bytes, %llu needed", k, (unsigned long long)args[k].bytes, (unsigned long long)q.n * 4);
  if (!writable(args[3])) return fail(VRHI_ERR_INVALID, "fused_map: output buffer is read-only (class %s)", vrhi_arg_class_name(args[3].buf_cls));
  const uint64_t n4 = q.n / 4;
  const int sms = st->dev->prop.multiProcessorCount;
  uint64_t want = (n4 + 255) / 256;
  // One wave: as many blocks as are resident at once.  A grid that spills into a second, partly filled
  // wave costs up to 20 % (measured: 5 blocks per SM 0.62 ms, 6 blocks 0.76 ms, 8 blocks 0.66 ms, 10 blocks 0.62 ms).
  static int resident = 0;
  if (resident == 0) {
    int nb = 0;
    VRHI_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fused_map_kernel<2>, 256, 0));
    resident = nb > 0 ? nb : 1;
  }
  uint64_t cap = (uint64_t)sms * resident;
  static const int env_blocks = env_int("VRHI_MAP_BLOCKS_PER_SM", 1, 32, 0);  // tuning aid
  if (env_blocks) cap = (uint64_t)sms * env_blocks;
  unsigned grid = (unsigned)(want < cap ? (want ? want : 1) : cap);
  fused_map_kernel<2><<<grid, 256, 0, st->s>>>(
      (const float4 *)args[0].ptr, (const float4 *)args[1].ptr, (const float4 *)args[2].ptr, (float4 *)args[3].ptr, n4, q.n,
      (const float *)args[0].ptr, (const float *)args[1].ptr, (const float *)args[2].ptr, (float *)args[3].ptr);
  return post_launch(st, "fused_map");
}

// ---------------------------------------------------------------------------------------------
// Generic fused tape.  The caller's tape is in SSA form (instruction t defines value
// n_inputs + t).  The host turns it into a short physical program over SLOTS: every input, every
// constant and every intermediate value lives in a slot (one float4 per element group per
// thread, in shared memory, laid out [slot][group][thread] so that accesses are conflict free);
// slots are assigned by a linear scan over live ranges and constants are written once per
// kernel.  The kernel handles G groups (4*G elements) per thread per trip, so that decoding an
// instruction is paid once per 4*G elements, and dispatches in two levels (operation class, then
// operation) with branches that are uniform across the CTA.  Long chains are bound by instruction
// issue and shared-memory traffic rather than by HBM; the specialised kernels above exist for the
// chains that matter most.

constexpr int kTapeThreads = 128;
constexpr int kTapeSlotBytes = 44 * 1024;  // slots; the staged programs (4 KiB) share the default 48 KiB limit

enum { CLS_BINARY = 0, CLS_UNARY = 1, CLS_TRANS = 2, CLS_FMA = 3 };

// One physical instruction: 32 bytes, word-sized fields (no byte unpacking on the device).
// dst / a / b / c are slot indices.
struct TapeInstrDev {
  uint32_t cls, op, dst, a, b, c, pad0, pad1;
};

struct TapeDev {
  uint32_t n_inputs, n_outputs, n_instr, n_slots, n_consts;
  uint32_t row_vector_mask, col_vector_mask, scalar_mask;
  uint8_t in_slot[VRHI_TAPE_MAX_INPUTS];   // 255: the input is never read
  uint8_t out_slot[VRHI_TAPE_MAX_OUTPUTS];
  uint8_t const_slot[16];
  float const_val[16];
  TapeInstrDev instr[VRHI_TAPE_MAX_INSTR];
  const float *in[VRHI_TAPE_MAX_INPUTS];
  float *out[VRHI_TAPE_MAX_OUTPUTS];
  uint64_t rows, cols;
};

#define TAPE_U(EXPR)                                                                              \
  _Pragma("unroll") for (int g = 0; g < G; ++g) {                                                 \
    const float4 va = pa[g * kTapeThreads];                                                       \
    float4 r;                                                                                     \
    { const float a = va.x; r.x = (EXPR); } { const float a = va.y; r.y = (EXPR); }               \
    { const float a = va.z; r.z = (EXPR); } { const float a = va.w; r.w = (EXPR); }               \
    pd[g * kTapeThreads] = r;                                                                     \
  }
#define TAPE_B(EXPR)                                                                              \
  _Pragma("unroll") for (int g = 0; g < G; ++g) {                                                 \
    const float4 va = pa[g * kTapeThreads], vb = pb[g * kTapeThreads];                            \
    float4 r;                                                                                     \
    { const float a = va.x, b = vb.x; r.x = (EXPR); } { const float a = va.y, b = vb.y; r.y = (EXPR); } \
    { const float a = va.z, b = vb.z; r.z = (EXPR); } { const float a = va.w, b = vb.w; r.w = (EXPR); } \
    pd[g * kTapeThreads] = r;                                                                     \
  }

// Executes the program on the G float4 groups held in the slots of this thread.
// `mine` points at this thread's element of slot 0, group 0.
// `prog` is the CTA's copy of the program in shared memory (broadcast reads, short latency).
template <int G>
__device__ __forceinline__ void tape_run(const TapeInstrDev *prog, uint32_t n_instr, float4 *mine) {
  constexpr int kSlotStride = G * kTapeThreads;  // float4s between consecutive slots
  TapeInstrDev I = prog[0];
  for (uint32_t t = 0; t < n_instr; ++t) {
    const TapeInstrDev cur = I;
    I = prog[t + 1 < n_instr ? t + 1 : t];  // fetch the next instruction while this one executes
    const float4 *pa = mine + cur.a * kSlotStride;
    const float4 *pb = mine + cur.b * kSlotStride;
    float4 *pd = mine + cur.dst * kSlotStride;
    switch (cur.cls) {
      case CLS_BINARY:
        switch (cur.op) {
          case VRHI_T_ADD: TAPE_B(a + b); break;
          case VRHI_T_SUB: TAPE_B(a - b); break;
          case VRHI_T_MUL: TAPE_B(a * b); break;
          case VRHI_T_DIV: TAPE_B(a / b); break;
          case VRHI_T_MAX: TAPE_B(fmaxf(a, b)); break;
          case VRHI_T_MIN: TAPE_B(fminf(a, b)); break;
          default: TAPE_B(a == b ? 1.f : 0.f); break;  // VRHI_T_EQ
        }
        break;
      case CLS_UNARY:
        switch (cur.op) {
          case VRHI_T_NEG: TAPE_U(-a); break;
          case VRHI_T_ABS: TAPE_U(fabsf(a)); break;
          case VRHI_T_SQUARE: TAPE_U(a * a); break;
          case VRHI_T_RELU: TAPE_U(fmaxf(a, 0.0f)); break;
          case VRHI_T_SIGN: TAPE_U((a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f)); break;
          case VRHI_T_STEP: TAPE_U(a > 0.f ? 1.f : 0.f); break;
          default: TAPE_U(a); break;  // VRHI_T_CONST as an output: copy of its slot
        }
        break;
      case CLS_TRANS:
        switch (cur.op) {
          case VRHI_T_SQRT: TAPE_U(sqrtf(a)); break;
          case VRHI_T_RSQRT: TAPE_U(1.0f / sqrtf(a)); break;
          case VRHI_T_RECIP: TAPE_U(1.0f / a); break;
          case VRHI_T_EXP: TAPE_U(expf(a)); break;
          case VRHI_T_LOG: TAPE_U(logf(a)); break;
          case VRHI_T_TANH: TAPE_U(tanhf(a)); break;
          case VRHI_T_SIGMOID: TAPE_U(sigmoid_accurate(a)); break;
          case VRHI_T_COS: TAPE_U(cosf(a)); break;
          default: TAPE_U(sinf(a)); break;  // VRHI_T_SIN
        }
        break;
      default: {  // CLS_FMA
        const float4 *pc = mine + cur.c * kSlotStride;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 va = pa[g * kTapeThreads], vb = pb[g * kTapeThreads], vc = pc[g * kTapeThreads];
          pd[g * kTapeThreads] = make_float4(fmaf(va.x, vb.x, vc.x), fmaf(va.y, vb.y, vc.y), fmaf(va.z, vb.z, vc.z), fmaf(va.w, vb.w, vc.w));
        }
        break;
      }
    }
  }
}

template <int G>
__device__ __forceinline__ void tape_fill_consts(const TapeDev &T, float4 *mine) {
  for (uint32_t k = 0; k < T.n_consts; ++k) {
    const float v = T.const_val[k];
#pragma unroll
    for (int g = 0; g < G; ++g) mine[(T.const_slot[k] * G + g) * kTapeThreads] = make_float4(v, v, v, v);
  }
}

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Vector path: cols % 4 == 0.  blockIdx.x walks column groups of kTapeThreads float4s,
// blockIdx.y strides over rows (G rows per trip), so a broadcast row vector is loaded once per thread.
//
// Inputs are double buffered: slots [0, NI) hold the inputs of even trips, slots [NI, 2*NI) those of
// odd trips, and the program exists in two copies that differ only in which of the two ranges they
// name.  While the program of one trip runs, the full-size inputs of the next trip are already on
// their way from HBM into the other range (cp.async, 16 bytes per thread per input per row, no
// registers held), so the memory latency of a trip hides behind the arithmetic of the previous one.
template <int G>
__global__ void __launch_bounds__(kTapeThreads, 8) map_tape_vec_kernel(const __grid_constant__ TapeDev T) {
  extern __shared__ float4 slots[];
  const int tid = threadIdx.x;
  float4 *mine = slots + tid;
  __shared__ TapeInstrDev prog[2][VRHI_TAPE_MAX_INSTR];
  const uint32_t NI = T.n_inputs;
  auto other = [NI](uint32_t s) -> uint32_t { return s < NI ? s + NI : (s < 2 * NI ? s - NI : s); };
  for (uint32_t k = tid; k < T.n_instr; k += kTapeThreads) {
    TapeInstrDev I = T.instr[k];
    prog[0][k] = I;
    I.dst = other(I.dst); I.a = other(I.a); I.b = other(I.b); I.c = other(I.c);
    prog[1][k] = I;
  }
  tape_fill_consts<G>(T, mine);
  __syncthreads();
  const uint64_t cols4 = T.cols / 4;
  const uint64_t cg = (uint64_t)blockIdx.x * kTapeThreads + tid;
  const bool in_range = cg < cols4;
  const uint32_t bcast_mask = T.row_vector_mask | T.col_vector_mask | T.scalar_mask;
  float4 rowvec[VRHI_TAPE_MAX_INPUTS];
#pragma unroll
  for (int k = 0; k < VRHI_TAPE_MAX_INPUTS; ++k) {
    rowvec[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < (int)NI && ((T.row_vector_mask >> k) & 1u) && in_range)
      rowvec[k] = reinterpret_cast<const float4 *>(T.in[k])[cg];
    if (k < (int)NI && ((T.scalar_mask >> k) & 1u)) {
      const float s = T.in[k][0];
      rowvec[k] = make_float4(s, s, s, s);
    }
  }
  // asynchronous loads of the full-size inputs of the trip that starts at row r0 into range `stage`
  auto prefetch = [&](uint64_t r0, uint32_t stage) {
    if (in_range && r0 < T.rows) {
      for (uint32_t k = 0; k < NI; ++k) {
        if (((bcast_mask >> k) & 1u) || T.in_slot[k] == 255) continue;
#pragma unroll
        for (int g = 0; g < G; ++g)
          if (r0 + g < T.rows)
            cp_async_16(mine + ((k + stage * NI) * G + g) * kTapeThreads, reinterpret_cast<const float4 *>(T.in[k]) + (r0 + g) * cols4 + cg);
      }
    }
    cp_async_commit();
  };
  const uint64_t step = (uint64_t)gridDim.y * G;
  uint64_t r0 = (uint64_t)blockIdx.y * G;
  uint32_t stage = 0;
  prefetch(r0, 0);
  for (; r0 < T.rows; r0 += step, stage ^= 1u) {
    prefetch(r0 + step, stage ^ 1u);  // commits a (possibly empty) group, so the wait below is uniform
    cp_async_wait<1>();                // everything but the group just committed has landed
    // broadcast inputs are written from registers into the current range
    for (uint32_t k = 0; k < NI; ++k) {
      if (!((bcast_mask >> k) & 1u) || T.in_slot[k] == 255) continue;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float4 v = rowvec[k];
        if (((T.col_vector_mask >> k) & 1u) && r0 + g < T.rows) {
          const float s = T.in[k][r0 + g];
          v = make_float4(s, s, s, s);
        }
        mine[((k + stage * NI) * G + g) * kTapeThreads] = v;
      }
    }
    tape_run<G>(prog[stage], T.n_instr, mine);
    if (in_range) {
#pragma unroll
      for (int k = 0; k < VRHI_TAPE_MAX_OUTPUTS; ++k)
        if (k < (int)T.n_outputs) {
          const uint32_t os = stage ? other(T.out_slot[k]) : T.out_slot[k];
#pragma unroll
          for (int g = 0; g < G; ++g)
            if (r0 + g < T.rows)
              st_stream(reinterpret_cast<float4 *>(T.out[k]) + (r0 + g) * cols4 + cg, mine[(os * G + g) * kTapeThreads]);
        }
    }
  }
  cp_async_wait<0>();
}

// Scalar path for any shape: one element per thread per trip (lane .x of the float4 slot).
__global__ void __launch_bounds__(kTapeThreads) map_tape_scalar_kernel(const __grid_constant__ TapeDev T) {
  extern __shared__ float4 slots[];
  const int tid = threadIdx.x;
  float4 *mine = slots + tid;
  __shared__ TapeInstrDev prog[VRHI_TAPE_MAX_INSTR];
  for (uint32_t k = tid; k < T.n_instr; k += kTapeThreads) prog[k] = T.instr[k];
  tape_fill_consts<1>(T, mine);
  __syncthreads();
  const uint64_t n = T.rows * T.cols;
  const uint64_t stride = (uint64_t)gridDim.x * kTapeThreads;
  for (uint64_t base = (uint64_t)blockIdx.x * kTapeThreads; base < n; base += stride) {
    const uint64_t e = base + tid;
    const bool in_range = e < n;
    const uint64_t col = in_range ? e % T.cols : 0;
    for (uint32_t k = 0; k < T.n_inputs; ++k) {
      if (T.in_slot[k] == 255) continue;
      float v = 0.f;
      if (in_range) {
        if ((T.row_vector_mask >> k) & 1u) v = T.in[k][col];
        else if ((T.col_vector_mask >> k) & 1u) v = T.in[k][e / T.cols];
        else if ((T.scalar_mask >> k) & 1u) v = T.in[k][0];
        else v = T.in[k][e];
      }
      slots[T.in_slot[k] * kTapeThreads + tid] = make_float4(v, v, v, v);
    }
    tape_run<1>(prog, T.n_instr, mine);
    if (in_range)
      for (uint32_t k = 0; k < T.n_outputs; ++k) T.out[k][e] = slots[T.out_slot[k] * kTapeThreads + tid].x;
  }
}

// What both execution paths require of a tape: known opcodes, operands defined before use, outputs that exist.
static int validate_tape(const vrhi_tape_params &q) {
  const int NI = (int)q.n_inputs, NT = (int)q.n_instr;
  for (int t = 0; t < NT; ++t) {
    const vrhi_tape_instr &I = q.instr[t];
    if (I.op >= VRHI_T_OPCOUNT) return fail(VRHI_ERR_INVALID, "map_tape: instruction %d has unknown opcode %u", t, I.op);
    const int ar = tape_arity(I.op);
    const uint16_t src[3] = {I.a, I.b, I.c};
    for (int s = 0; s < ar; ++s)
      if (src[s] >= NI + t) return fail(VRHI_ERR_INVALID, "map_tape: instruction %d reads value %u before it is defined", t, src[s]);
  }
  for (uint32_t k = 0; k < q.n_outputs; ++k)
    if ((int)q.out_value[k] >= NI + NT) return fail(VRHI_ERR_INVALID, "map_tape: output %u names value %u, which does not exist", k, q.out_value[k]);
  return VRHI_OK;
}

// SSA tape -> physical program (see the comment at the top of this section).
static int plan_tape(const vrhi_tape_params &q, TapeDev *T, int max_slots) {
  const int NI = (int)q.n_inputs, NT = (int)q.n_instr, NV = NI + NT;
  constexpr int MAXV = VRHI_TAPE_MAX_INPUTS + VRHI_TAPE_MAX_INSTR;
  bool is_const[MAXV] = {}, is_output[MAXV] = {};
  int last_use[MAXV], slot_of[MAXV];
  for (int v = 0; v < NV; ++v) { last_use[v] = -1; slot_of[v] = -1; }
  for (int t = 0; t < NT; ++t) {
    const vrhi_tape_instr &I = q.instr[t];
    if (I.op >= VRHI_T_OPCOUNT) return fail(VRHI_ERR_INVALID, "map_tape: instruction %d has unknown opcode %u", t, I.op);
    const int ar = tape_arity(I.op);
    const uint16_t src[3] = {I.a, I.b, I.c};
    for (int s = 0; s < ar; ++s) {
      if (src[s] >= NI + t) return fail(VRHI_ERR_INVALID, "map_tape: instruction %d reads value %u before it is defined", t, src[s]);
      last_use[src[s]] = t;
    }
    if (I.op == VRHI_T_CONST) is_const[NI + t] = true;
  }
  for (uint32_t k = 0; k < q.n_outputs; ++k) {
    if ((int)q.out_value[k] >= NV) return fail(VRHI_ERR_INVALID, "map_tape: output %u names value %u, which does not exist", k, q.out_value[k]);
    is_output[q.out_value[k]] = true;
  }
  bool busy[64] = {};
  int n_slots = 0;
  auto take = [&]() -> int {
    for (int s = 0; s < max_slots && s < 64; ++s)
      if (!busy[s]) { busy[s] = true; if (s + 1 > n_slots) n_slots = s + 1; return s; }
    return -1;
  };
  const char *too_many = "map_tape: more than %d values (inputs, constants, intermediates) live at once";
  // inputs own slots 0..NI-1; slots NI..2*NI-1 are the second input buffer of the vector kernel
  // and are never handed to intermediates (see map_tape_vec_kernel)
  for (int k = 0; k < NI; ++k) {
    int s = take();
    if (s != k) return fail(VRHI_ERR_UNSUPPORTED, too_many, max_slots);
    slot_of[k] = s;
    T->in_slot[k] = (last_use[k] < 0 && !is_output[k]) ? 255 : (uint8_t)s;
  }
  for (int k = 0; k < NI; ++k)
    if (take() != NI + k) return fail(VRHI_ERR_UNSUPPORTED, too_many, max_slots);
  // constants that are read hold a slot for the whole kernel (written once, before the first trip);
  // equal constants share one
  T->n_consts = 0;
  for (int t = 0; t < NT; ++t) {
    const int v = NI + t;
    if (!is_const[v] || (last_use[v] < 0 && !is_output[v])) continue;
    int found = -1;
    for (uint32_t k = 0; k < T->n_consts; ++k)
      if (memcmp(&T->const_val[k], &q.instr[t].imm, sizeof(float)) == 0) found = (int)k;
    if (found < 0) {
      if (T->n_consts >= 16) return fail(VRHI_ERR_UNSUPPORTED, "map_tape: more than 16 distinct constants");
      int s = take();
      if (s < 0) return fail(VRHI_ERR_UNSUPPORTED, too_many, max_slots);
      found = (int)T->n_consts++;
      T->const_slot[found] = (uint8_t)s;
      T->const_val[found] = q.instr[t].imm;
    }
    slot_of[v] = T->const_slot[found];
  }
  int NP = 0;
  for (int t = 0; t < NT; ++t) {
    const vrhi_tape_instr &I = q.instr[t];
    const int v = NI + t;
    if (I.op == VRHI_T_CONST) continue;
    const int ar = tape_arity(I.op);
    const int src[3] = {I.a, I.b, I.c};
    TapeInstrDev D{};
    D.op = I.op;
    D.cls = ar == 3 ? CLS_FMA : ar == 2 ? CLS_BINARY
            : (I.op == VRHI_T_NEG || I.op == VRHI_T_ABS || I.op == VRHI_T_SQUARE || I.op == VRHI_T_RELU || I.op == VRHI_T_SIGN || I.op == VRHI_T_STEP) ? CLS_UNARY
                                                                                                                                                     : CLS_TRANS;
    D.a = (uint32_t)slot_of[src[0]];
    D.b = ar >= 2 ? (uint32_t)slot_of[src[1]] : D.a;
    D.c = ar >= 3 ? (uint32_t)slot_of[src[2]] : D.a;
    // operands whose last use is here release their slot before the result is placed (a result
    // may overwrite its own operand: each thread reads its elements before it writes them)
    for (int s = 0; s < ar; ++s)
      if (!is_const[src[s]] && !is_output[src[s]] && last_use[src[s]] == t && slot_of[src[s]] >= 0) busy[slot_of[src[s]]] = false;
    int d = take();
    if (d < 0) return fail(VRHI_ERR_UNSUPPORTED, too_many, max_slots);
    slot_of[v] = d;
    D.dst = (uint32_t)d;
    if (last_use[v] < 0 && !is_output[v]) busy[d] = false;  // dead value
    T->instr[NP++] = D;
  }
  for (uint32_t k = 0; k < q.n_outputs; ++k) T->out_slot[k] = (uint8_t)slot_of[q.out_value[k]];
  T->n_instr = (uint32_t)NP;
  T->n_slots = (uint32_t)n_slots;
  return VRHI_OK;
}

int launch_map_tape(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_tape_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (q.n_inputs > VRHI_TAPE_MAX_INPUTS || q.n_outputs == 0 || q.n_outputs > VRHI_TAPE_MAX_OUTPUTS || q.n_instr > VRHI_TAPE_MAX_INSTR)
    return fail(VRHI_ERR_INVALID, "map_tape: %u inputs / %u outputs / %u instructions outside the limits (%d / 1..%d / %d)", q.n_inputs, q.n_outputs, q.n_instr, VRHI_TAPE_MAX_INPUTS, VRHI_TAPE_MAX_OUTPUTS, VRHI_TAPE_MAX_INSTR);
  if (n_args != (int)(q.n_inputs + q.n_outputs)) return fail(VRHI_ERR_INVALID, "map_tape: %d arguments passed, tape declares %u inputs + %u outputs", n_args, q.n_inputs, q.n_outputs);
  uint64_t n = 0;
  VRHI_TRY(element_count(q.rows, q.cols, "map_tape", &n));
  if (n == 0) return VRHI_OK;
  if ((q.row_vector_mask & q.col_vector_mask) | (q.row_vector_mask & q.scalar_mask) | (q.col_vector_mask & q.scalar_mask))
    return fail(VRHI_ERR_INVALID, "map_tape: an input is marked with more than one broadcast shape");
  VRHI_TRY(validate_tape(q));
  TapeDev T{};
  T.n_inputs = q.n_inputs; T.n_outputs = q.n_outputs;
  T.row_vector_mask = q.row_vector_mask; T.col_vector_mask = q.col_vector_mask; T.scalar_mask = q.scalar_mask;
  T.rows = q.rows; T.cols = q.cols;
  for (uint32_t k = 0; k < q.n_inputs; ++k) {
    uint64_t need = ((q.row_vector_mask >> k) & 1u) ? q.cols * 4 : ((q.col_vector_mask >> k) & 1u) ? q.rows * 4 : ((q.scalar_mask >> k) & 1u) ? 4 : n * 4;
    if (args[k].bytes < need) return fail(VRHI_ERR_SIZE, "map_tape: input %u holds %llu bytes, %llu needed", k, (unsigned long long)args[k].bytes, (unsigned long long)need);
    T.in[k] = (const float *)args[k].ptr;
  }
  for (uint32_t k = 0; k < q.n_outputs; ++k) {
    const ArgView &o = args[q.n_inputs + k];
    const uint64_t out_bytes = ((q.colsum_mask >> k) & 1u) ? q.cols * 4 : n * 4;
    if (o.bytes < out_bytes) return fail(VRHI_ERR_SIZE, "map_tape: output %u holds %llu bytes, %llu needed", k, (unsigned long long)o.bytes, (unsigned long long)out_bytes);
    if (!writable(o)) return fail(VRHI_ERR_INVALID, "map_tape: output %u is read-only (class %s)", k, vrhi_arg_class_name(o.buf_cls));
    T.out[k] = (float *)o.ptr;
  }
  // The tape compiled to a kernel of its own where that is possible (values in registers, HBM-bound);
  // the interpreter below otherwise.  Both compute the same bits.
  {
    const int rc = tape_jit_launch(st, q, T.in, T.out);
    if (rc == VRHI_OK) return post_launch(st, "map_tape (compiled)");
    if (rc != 1) return rc;
    if (q.colsum_mask) return fail(VRHI_ERR_UNSUPPORTED, "map_tape: column-summed outputs need the compiled path (run-time compiler present, columns a multiple of 4, 16-byte aligned arrays)");
  }
  const int slot_capacity = kTapeSlotBytes / (kTapeThreads * (int)sizeof(float4));  // 24 slots of one group
  VRHI_TRY(plan_tape(q, &T, slot_capacity));
  const int sms = st->dev->prop.multiProcessorCount;
  const uint32_t ns = T.n_slots ? T.n_slots : 1;
  if (q.cols % 4 == 0) {
    // two row groups per thread when the slots of both fit in 48 KiB of shared memory and there are rows to pair
    const int G = (ns * 2 <= (uint32_t)slot_capacity && q.rows >= 2) ? 2 : 1;
    const size_t smem = (size_t)ns * G * kTapeThreads * sizeof(float4);
    uint64_t cols4 = q.cols / 4;
    uint64_t gx = (cols4 + kTapeThreads - 1) / kTapeThreads;
    if (gx > 0x7fffffffull) return fail(VRHI_ERR_UNSUPPORTED, "map_tape: too many columns");
    uint64_t target = (uint64_t)sms * 8;
    uint64_t gy = (target + gx - 1) / gx;
    uint64_t row_groups = (q.rows + G - 1) / G;
    if (gy > row_groups) gy = row_groups;
    if (gy > 65535) gy = 65535;
    if (gy == 0) gy = 1;
    dim3 grid((unsigned)gx, (unsigned)gy);
    if (G == 2) map_tape_vec_kernel<2><<<grid, kTapeThreads, smem, st->s>>>(T);
    else map_tape_vec_kernel<1><<<grid, kTapeThreads, smem, st->s>>>(T);
  } else {
    const size_t smem = (size_t)ns * kTapeThreads * sizeof(float4);
    uint64_t want = (n + kTapeThreads - 1) / kTapeThreads;
    uint64_t cap = (uint64_t)sms * 8;
    map_tape_scalar_kernel<<<(unsigned)(want < cap ? want : cap), kTapeThreads, smem, st->s>>>(T);
  }
  return post_launch(st, "map_tape");
}

}  // namespace vrhi
