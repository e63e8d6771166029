// Escape-time map, regrouping kernel: two pixels per lane in packed binary32 pairs (sm_100a).
//
// Loop rules as in k_escape.cu (fractal.py:11-25): test before update, count the updates, square
// as (z0*z0 - z1*z1, (z1*z0)*2).  Accepted parameters: test "a+b > bound" with bound >= 4,
// |c| <= 1.5 (Mandelbrot pixels with a larger constant are finished at intake), max_iter >= 64.
//
// Iteration counts inside a warp differ by orders of magnitude near the set, so one pixel per lane
// with a test on every step leaves most lanes idle (about 36 % lane efficiency on the 16384^2
// Julia workload) and spends 11 issue slots per step.  This kernel keeps the slots busy:
//
//  * UNCHECKED BLOCKS.  A slot runs U updates with no test and no counter (six arithmetic
//    operations per update).  One test at the end decides whether the whole block was valid.  That
//    is exact because, for bound >= 4 and |c| <= 1.5, escape is monotonic even in binary32: once
//    a+b > bound then |z'| >= |z|^2 - |c| > 1.2|z|, so every later a+b is larger still, or Inf/NaN,
//    and the test is written !(s <= bound) so that NaN counts as escaped.  A slot whose block failed
//    the test (or would pass max_iter) is put back on its checkpoint and marked "finishing".
//  * CHECKED BLOCKS.  When at least T slots are finishing or empty, the warp runs one block of U
//    steps with the test and the counter on every step; slots still in flight simply advance,
//    finishing slots find their exact count.  Finished pixels are stored and their slots freed.
//  * POOL.  Freed slots are refilled from a per-warp ring in shared memory.  The ring is fed by
//    INTAKE: 64 fresh pixels of a stolen tile run K checked steps in lock step (most pixels of the
//    far exterior end there and are stored coalesced); survivors are pushed to the ring with their
//    state.  Long-lived pixels therefore share warps with other long-lived pixels.
//  * WORK STEALING.  Warps pull batches of up to 24 tiles (1536 pixels of one row) from a global
//    counter.  Nothing here waits on another warp or block: no spin loops, no barriers.
//
// TWO PIXELS PER LANE.  Every lane carries two slots, and all arithmetic on them is issued as packed
// instructions (fma/add/sub .rn.f32x2), one instruction for both.  On this GPU an SM sub-partition
// issues one instruction per clock and its binary32 pipe retires 32 lane-operations per clock.
// With one pixel per lane the six arithmetic instructions of an update fill the issue slot on
// every clock, and every test, counter, ballot and address computation costs a slot the arithmetic
// cannot use (measured: 36 % of all issued instructions).  A packed instruction occupies the pipe
// for two clocks but the issue slot for one, so part of the bookkeeping of this warp and of the
// other resident warps runs in the slots between.  Measured on B200, 16384^2 Julia image: 2.49 ms
// with one pixel per lane, 2.17 ms with two; 699 M -> 465 M issued instructions on the 8192^2 image.
//
// Exactness.  A packed operation rounds each half exactly like the scalar operation, so the counts
// are the same bits as the one-pixel-per-lane kernel and the CPU statement.  One trap: the
// assembler contracts mul.rn.f32x2 followed by add/sub.rn.f32x2 into a fused multiply-add (it does
// so even through fma(x, y, -0.0) with a literal -0.0), which changes the rounding of
// (zr*zr - zi*zi).  Every product here is therefore fma(x, y, nz) with nz = -0.0 read from the
// kernel parameters, a value the assembler cannot see: x*y + (-0.0) is x*y rounded once, sign of
// zero included, and an fma feeding an add is never contracted further.
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "escape_common.cuh"

namespace vrhi {

typedef unsigned long long f32x2;  // two binary32 values in one 64-bit register; "lo" is slot 0

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 neg2(f32x2 a) { return a ^ 0x8000000080000000ull; }
// lo half from `n` where c0 holds, else from `o`; hi half likewise with c1
__device__ __forceinline__ f32x2 select2(bool c0, bool c1, f32x2 n, f32x2 o) {
  float nl, nh, ol, oh;
  unpack2(n, nl, nh);
  unpack2(o, ol, oh);
  return pack2(c0 ? nl : ol, c1 ? nh : oh);
}

// The step primitives of escape_common.cuh on pairs; `nz` is the invisible -0.0 (see the top).
template <int MODE>
__device__ __forceinline__ void pair_squares(f32x2 zr, f32x2 zi, f32x2 nz, f32x2 &a, f32x2 &b) {
  if (MODE == VRHI_ESCAPE_EXACT) { a = fma2(zr, zr, nz); b = fma2(zi, zi, nz); }
}
template <int MODE>
__device__ __forceinline__ f32x2 pair_norm2(f32x2 zr, f32x2 zi, f32x2 a, f32x2 b, f32x2 nz) {
  if (MODE == VRHI_ESCAPE_EXACT) return add2(a, b);
  return fma2(zi, zi, fma2(zr, zr, nz));
}
template <int MODE>
__device__ __forceinline__ void pair_advance(f32x2 &zr, f32x2 &zi, f32x2 &a, f32x2 &b, f32x2 cr, f32x2 ci, f32x2 nz, f32x2 two) {
  if (MODE == VRHI_ESCAPE_EXACT) {
    const f32x2 t = fma2(zr, zi, nz);
    zi = fma2(two, t, ci);
    zr = add2(sub2(a, b), cr);
    a = fma2(zr, zr, nz);
    b = fma2(zi, zi, nz);
  } else {
    const f32x2 nzi = fma2(add2(zr, zr), zi, ci);
    zr = fma2(zr, zr, fma2(neg2(zi), zi, cr));
    zi = nzi;
  }
}

constexpr int kPairPool = 128;  // pool entries per warp: a refill wants up to 64, an intake trip adds up to 64

// U = updates per block, T = waiting slots (of 64) that trigger a checked block, K = checked steps
// a fresh pixel gets before it is pooled, EX = bit k set: intake stops before step k when every
// pixel of the tile has ended, NBLK = unchecked blocks between two counts of the waiting slots
template <int KIND, int OUT, int U, int T, int K, int MODE, bool WIRE, int EX, int NBLK>
__global__ void __launch_bounds__(256, 4) escape_pair_kernel(EscapeDev p, void *image, uint32_t *work_counter, uint16_t *wire) {
  constexpr bool PER_PIXEL_C = (KIND == VRHI_ESCAPE_MANDELBROT);
  begin_overlap();
  __shared__ float4 s_pool[8][kPairPool];  // zr, zi, pixel index, count: one 16-byte access per entry
  __shared__ float2 s_c[PER_PIXEL_C ? 8 : 1][PER_PIXEL_C ? kPairPool : 1];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  const uint32_t FULL = 0xffffffffu;
  float4 *pool = s_pool[warp];
  float2 *poolc = s_c[PER_PIXEL_C ? warp : 0];
  const float bound = p.bound, x0 = p.x0, dx = p.dx, color_scale = p.color_scale;
  const uint32_t max_iter = p.max_iter, width = p.width;
  const bool transposed = p.transposed != 0;
  const uint32_t fast_limit = max_iter - (uint32_t)U;  // the host guarantees max_iter >= U
  const f32x2 NZ = pack2(p.neg_zero, p.neg_zero), TWO = pack2(2.0f, 2.0f);

  // warp-uniform state
  uint32_t pool_head = 0, pool_tail = 0, pool_n = 0;
  bool fresh = true;
  uint32_t tile = 0, tile_end = 0, row_base = 0;  // tiles of 64 pixels
  float row_y = 0.f;
  // lane state: slot 0 in the low halves, slot 1 in the high halves
  f32x2 ZR = 0, ZI = 0, A = 0, B = 0, CR = pack2(p.cr, p.cr), CI = pack2(p.ci, p.ci);
  uint32_t cnt0 = 0, cnt1 = 0, idx0 = 0, idx1 = 0;
  bool occ0 = false, occ1 = false;  // the slot holds a pixel
  bool run0 = false, run1 = false;  // ... that may go through unchecked blocks (occ && !run: finishing)

  auto finish = [&](uint32_t pix, uint32_t count) {
    store_count<OUT>(image, (size_t)pix, count, color_scale);
    if (WIRE) store_wire(wire, p.bytes, (size_t)pix, count);
  };

  auto intake = [&]() {
    if (tile >= tile_end) {
      uint32_t batch = 0;
      if (lane == 0) batch = atomicAdd(work_counter, 1u);
      batch = __shfl_sync(FULL, batch, 0);
      if (batch >= p.n_batches) { fresh = false; return; }
      const uint32_t k = batch / p.batches_per_row;
      tile = (batch - k * p.batches_per_row) * p.batch_tiles;
      const uint32_t r = middle_out(k, p.rows_owned);  // expensive rows first: their long pixels end under cover of the rest
      tile_end = min(tile + p.batch_tiles, p.tiles_per_row);
      const uint32_t j = owned_row_to_image_row(p, r);
      row_y = __fadd_rn(p.y0, __fmul_rn((float)j, p.dy));
      row_base = j * width;
    }
    const uint32_t i0 = tile * 64u + lane, i1 = i0 + 32u;
    ++tile;
    const bool valid0 = i0 < width, valid1 = i1 < width;
    const f32x2 X = pack2(__fadd_rn(x0, __fmul_rn((float)i0, dx)), __fadd_rn(x0, __fmul_rn((float)i1, dx)));
    const f32x2 Y = pack2(row_y, row_y);
    const f32x2 RE = transposed ? Y : X, IM = transposed ? X : Y;
    f32x2 FZR, FZI, FCR, FCI;
    if (PER_PIXEL_C) { FZR = 0; FZI = 0; FCR = RE; FCI = IM; }
    else { FZR = RE; FZI = IM; FCR = CR; FCI = CI; }
    uint32_t fc0 = 0, fc1 = 0;
    bool l0 = valid0, l1 = valid1;
    f32x2 FA = 0, FB = 0;
    pair_squares<MODE>(FZR, FZI, NZ, FA, FB);
    // K steps with a test on each, straight-line: dead slots keep computing values nobody reads.
    // The host guarantees max_iter >= K: no cap test in here.
#pragma unroll
    for (int k = 0; k < K; ++k) {
      float s0, s1;
      unpack2(pair_norm2<MODE>(FZR, FZI, FA, FB, NZ), s0, s1);
      l0 = l0 && (s0 <= bound);
      l1 = l1 && (s1 <= bound);
      // most tiles lie far outside the set and die within two or three steps, all slots together
      if (((EX >> k) & 1) && k < K - 1 && !__any_sync(FULL, l0 || l1)) break;
      pair_advance<MODE>(FZR, FZI, FA, FB, FCR, FCI, NZ, TWO);
      fc0 += l0 ? 1u : 0u;
      fc1 += l1 ? 1u : 0u;
    }
    if (PER_PIXEL_C) {
      // pixels whose own constant is too large for unchecked blocks are finished here, step by step
      float c0r, c1r, c0i, c1i;
      unpack2(FCR, c0r, c1r);
      unpack2(FCI, c0i, c1i);
      bool slow0 = l0 && !(__fmaf_rn(c0r, c0r, __fmul_rn(c0i, c0i)) <= 2.25f);
      bool slow1 = l1 && !(__fmaf_rn(c1r, c1r, __fmul_rn(c1i, c1i)) <= 2.25f);
      while (__any_sync(FULL, slow0 || slow1)) {
        float s0, s1;
        unpack2(pair_norm2<MODE>(FZR, FZI, FA, FB, NZ), s0, s1);
        if (slow0 && (!(s0 <= bound) || fc0 >= max_iter)) { slow0 = false; l0 = false; }
        if (slow1 && (!(s1 <= bound) || fc1 >= max_iter)) { slow1 = false; l1 = false; }
        f32x2 NR = FZR, NI = FZI, NA = FA, NB = FB;
        pair_advance<MODE>(NR, NI, NA, NB, FCR, FCI, NZ, TWO);
        // only the slots being finished here move; survivors on their way to the pool keep their state
        FZR = select2(slow0, slow1, NR, FZR);
        FZI = select2(slow0, slow1, NI, FZI);
        if (MODE == VRHI_ESCAPE_EXACT) { FA = select2(slow0, slow1, NA, FA); FB = select2(slow0, slow1, NB, FB); }
        fc0 += slow0 ? 1u : 0u;
        fc1 += slow1 ? 1u : 0u;
      }
    }
    if (valid0 && !l0) finish(row_base + i0, fc0);
    if (valid1 && !l1) finish(row_base + i1, fc1);
    const uint32_t m0 = __ballot_sync(FULL, l0), m1 = __ballot_sync(FULL, l1);
    if (m0 | m1) {
      const uint32_t n0 = __popc(m0);
      float zr0, zr1, zi0, zi1;
      unpack2(FZR, zr0, zr1);
      unpack2(FZI, zi0, zi1);
      if (l0) {
        const uint32_t slot = (pool_head + __popc(m0 & lt_mask)) & (kPairPool - 1);
        pool[slot] = make_float4(zr0, zi0, __uint_as_float(row_base + i0), __uint_as_float(fc0));
        if (PER_PIXEL_C) { float cr0, cr1, ci0, ci1; unpack2(FCR, cr0, cr1); unpack2(FCI, ci0, ci1); poolc[slot] = make_float2(cr0, ci0); }
      }
      if (l1) {
        const uint32_t slot = (pool_head + n0 + __popc(m1 & lt_mask)) & (kPairPool - 1);
        pool[slot] = make_float4(zr1, zi1, __uint_as_float(row_base + i1), __uint_as_float(fc1));
        if (PER_PIXEL_C) { float cr0, cr1, ci0, ci1; unpack2(FCR, cr0, cr1); unpack2(FCI, ci0, ci1); poolc[slot] = make_float2(cr1, ci1); }
      }
      const uint32_t n = n0 + __popc(m1);
      pool_head = (pool_head + n) & (kPairPool - 1);
      pool_n += n;
      __syncwarp();
    }
  };

  // One block of U steps with the test on every step, straight-line: a slot that has stopped keeps
  // computing values nobody reads, only its counter is frozen.  CAP = false is used when no slot
  // can reach max_iter inside the block, which saves the counter comparisons.
  auto checked_block = [&](auto cap_tag) {
    constexpr bool CAP = decltype(cap_tag)::value;
    pair_squares<MODE>(ZR, ZI, NZ, A, B);  // finishing slots were put back on their checkpoint: refresh the squares
    bool live0 = occ0, live1 = occ1;
#pragma unroll
    for (int k = 0; k < U; ++k) {
      float s0, s1;
      unpack2(pair_norm2<MODE>(ZR, ZI, A, B, NZ), s0, s1);
      live0 = live0 && (s0 <= bound);
      live1 = live1 && (s1 <= bound);
      if (CAP) { live0 = live0 && (cnt0 < max_iter); live1 = live1 && (cnt1 < max_iter); }
      pair_advance<MODE>(ZR, ZI, A, B, CR, CI, NZ, TWO);
      cnt0 += live0 ? 1u : 0u;
      cnt1 += live1 ? 1u : 0u;
    }
    // the block made U tests and up to U updates; a slot whose unchecked block failed only at its
    // very last state needs the test of that state too (tests are idempotent)
    {
      float s0, s1;
      unpack2(pair_norm2<MODE>(ZR, ZI, A, B, NZ), s0, s1);
      live0 = live0 && (s0 <= bound);
      live1 = live1 && (s1 <= bound);
      if (CAP) { live0 = live0 && (cnt0 < max_iter); live1 = live1 && (cnt1 < max_iter); }
    }
    if (occ0 && !live0) finish(idx0, cnt0);
    if (occ1 && !live1) finish(idx1, cnt1);
    occ0 = live0; run0 = live0;  // a finishing slot always ends inside the block
    occ1 = live1; run1 = live1;
  };

  for (;;) {
    // ---- refill: feed the pool until every empty slot can be served, then hand out entries
    const uint32_t f0 = __ballot_sync(FULL, !occ0), f1 = __ballot_sync(FULL, !occ1);
    if (f0 | f1) {
      const uint32_t n0 = __popc(f0), need = n0 + __popc(f1);
      while (pool_n < need && fresh) intake();
      if (pool_n) {
        const uint32_t r0 = __popc(f0 & lt_mask), r1 = n0 + __popc(f1 & lt_mask);
        float zr0, zr1, zi0, zi1, cr0 = 0.f, cr1 = 0.f, ci0 = 0.f, ci1 = 0.f;
        unpack2(ZR, zr0, zr1);
        unpack2(ZI, zi0, zi1);
        if (PER_PIXEL_C) { unpack2(CR, cr0, cr1); unpack2(CI, ci0, ci1); }
        if (!occ0 && r0 < pool_n) {
          const uint32_t slot = (pool_tail + r0) & (kPairPool - 1);
          const float4 e = pool[slot];
          zr0 = e.x; zi0 = e.y; idx0 = __float_as_uint(e.z); cnt0 = __float_as_uint(e.w);
          if (PER_PIXEL_C) { const float2 c = poolc[slot]; cr0 = c.x; ci0 = c.y; }
          occ0 = true; run0 = true;
        }
        if (!occ1 && r1 < pool_n) {
          const uint32_t slot = (pool_tail + r1) & (kPairPool - 1);
          const float4 e = pool[slot];
          zr1 = e.x; zi1 = e.y; idx1 = __float_as_uint(e.z); cnt1 = __float_as_uint(e.w);
          if (PER_PIXEL_C) { const float2 c = poolc[slot]; cr1 = c.x; ci1 = c.y; }
          occ1 = true; run1 = true;
        }
        ZR = pack2(zr0, zr1);
        ZI = pack2(zi0, zi1);
        if (PER_PIXEL_C) { CR = pack2(cr0, cr1); CI = pack2(ci0, ci1); }
        pair_squares<MODE>(ZR, ZI, NZ, A, B);
        const uint32_t popped = min(need, pool_n);
        pool_tail = (pool_tail + popped) & (kPairPool - 1);
        pool_n -= popped;
        __syncwarp();
      }
    }
    uint32_t waiting = __popc(__ballot_sync(FULL, !run0)) + __popc(__ballot_sync(FULL, !run1));
    if (waiting == 64u && __ballot_sync(FULL, occ0 || occ1) == 0u) break;  // pool empty, no fresh tiles, nothing in flight
    // ---- unchecked blocks until enough slots want attention (all of them once nothing can be refilled)
    const uint32_t threshold = (!fresh && pool_n == 0) ? 64u : (uint32_t)T;
    while (waiting < threshold) {
#pragma unroll
      for (int nb = 0; nb < NBLK; ++nb) {
        const f32x2 CKR = ZR, CKI = ZI;
#pragma unroll
        for (int k = 0; k < U; ++k) pair_advance<MODE>(ZR, ZI, A, B, CR, CI, NZ, TWO);
        // slots that are not running (empty or finishing) computed garbage: they, and slots whose
        // block failed, go back to the checkpoint; a and b are refreshed below or by the checked block
        float s0, s1;
        unpack2(pair_norm2<MODE>(ZR, ZI, A, B, NZ), s0, s1);
        run0 = run0 && (s0 <= bound) && (cnt0 <= fast_limit);
        run1 = run1 && (s1 <= bound) && (cnt1 <= fast_limit);
        cnt0 += run0 ? (uint32_t)U : 0u;
        cnt1 += run1 ? (uint32_t)U : 0u;
        ZR = select2(run0, run1, ZR, CKR);
        ZI = select2(run0, run1, ZI, CKI);
        if (nb + 1 < NBLK) pair_squares<MODE>(ZR, ZI, NZ, A, B);
      }
      waiting = __popc(__ballot_sync(FULL, !run0)) + __popc(__ballot_sync(FULL, !run1));
    }
    // ---- one checked block: finishing slots find their exact count, the others just advance
    if (__any_sync(FULL, (occ0 && cnt0 > fast_limit) || (occ1 && cnt1 > fast_limit))) checked_block(std::true_type{});
    else checked_block(std::false_type{});
  }
  end_overlap();
}

// The shipped instantiation: U = 12, T = 16 of 64, K = 12 with exits before steps 2, 4, 6 and 8, two blocks
// between counts.  Sweeps on B200 (U = 6..24, T = 4..32, K = 4..16, one to four blocks between counts)
// stayed within 3 % of this point on the 16384^2 Julia image.

int launch_escape_pair(vrhi_stream_t *st, const vrhi_escape_params &q, const EscapeDev &p, int grid, int per_sm, bool pin, bool overlap,
                       void *image, uint32_t *counter, uint16_t *wire) {
  constexpr int U = 12, T = 16, K = 12, EX = 0x154, NBLK = 2;
#define PAIR(KIND, OUT, WIRE)                                                                                                        \
  do {                                                                                                                               \
    if (q.mode == VRHI_ESCAPE_EXACT) return launch_pinned(escape_pair_kernel<KIND, OUT, U, T, K, VRHI_ESCAPE_EXACT, WIRE, EX, NBLK>, grid, per_sm, st, p, image, counter, wire, pin, overlap); \
    return launch_pinned(escape_pair_kernel<KIND, OUT, U, T, K, VRHI_ESCAPE_FAST, WIRE, EX, NBLK>, grid, per_sm, st, p, image, counter, wire, pin, overlap);  \
  } while (0)
  if (wire) {
    if (q.kind == VRHI_ESCAPE_MANDELBROT) PAIR(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COUNT_U32, true);
    PAIR(VRHI_ESCAPE_JULIA, VRHI_OUT_COUNT_U32, true);
  }
  if (q.kind == VRHI_ESCAPE_MANDELBROT) {
    if (q.output == VRHI_OUT_COUNT_U32) PAIR(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COUNT_U32, false);
    if (q.output == VRHI_OUT_COUNT_U16) PAIR(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COUNT_U16, false);
    PAIR(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COLOR_F32, false);
  }
  if (q.output == VRHI_OUT_COUNT_U32) PAIR(VRHI_ESCAPE_JULIA, VRHI_OUT_COUNT_U32, false);
  if (q.output == VRHI_OUT_COUNT_U16) PAIR(VRHI_ESCAPE_JULIA, VRHI_OUT_COUNT_U16, false);
  PAIR(VRHI_ESCAPE_JULIA, VRHI_OUT_COLOR_F32, false);
#undef PAIR
}

}  // namespace vrhi
