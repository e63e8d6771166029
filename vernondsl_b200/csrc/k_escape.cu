// Escape-time map kernels (Mandelbrot / Julia), sm_100a.
//
// Loop rules follow fractal.py:18-25: every pixel is independent, the escape test comes before
// the update, the result counts the updates performed; the square is (z0*z0 - z1*z1, (z1*z0)*2)
// (fractal.py:11-13); coordinates come from the integer index at the pixel corner
// (fractal.py:20).
//
// EXACT mode reproduces these binary32 roundings and no others:
//     a = zr*zr; b = zi*zi; s = a+b; t = zr*zi; zi' = (t+t)+ci; zr' = (a-b)+cr
// (t+t)+ci is issued as fma(2, t, ci): 2*t is exact in binary32, so the fused form rounds the
// same real number once and gives the same bits with one instruction fewer.  Everything else uses
// __fmul_rn / __fadd_rn, which the compiler never contracts.
//
// This file holds the fully checked kernel: one pixel per lane, a test on every step.  It accepts
// every parameter combination and is the path of record for parameters the regrouping kernel
// cannot take.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "escape_common.cuh"

namespace vrhi {

template <int KIND, int MODE, int TEST, int OUT>
__global__ void __launch_bounds__(256) escape_checked_kernel(EscapeDev p, void *image, uint32_t *work_counter, uint16_t *wire) {
  const uint32_t lane = threadIdx.x & 31u;
  // work_counter == nullptr: batches are dealt to warps round-robin (small frames, where the
  // counter's reset would cost as much as the frame); otherwise warps pull batches from the counter
  uint32_t next = blockIdx.x * 8u + (threadIdx.x >> 5);
  for (;;) {
    uint32_t batch = next;
    if (work_counter) {
      if (lane == 0) batch = atomicAdd(work_counter, 1u);
      batch = __shfl_sync(0xffffffffu, batch, 0);
    } else {
      next += gridDim.x * 8u;
    }
    if (batch >= p.n_batches) break;
    const uint32_t r = batch / p.batches_per_row;
    const uint32_t tile0 = (batch - r * p.batches_per_row) * p.batch_tiles;
    const uint32_t tile1 = min(tile0 + p.batch_tiles, p.tiles_per_row);
    const uint32_t j = owned_row_to_image_row(p, r);
    const float y = __fadd_rn(p.y0, __fmul_rn((float)j, p.dy));
    const size_t row_base = (size_t)j * p.width;
    for (uint32_t tile = tile0; tile < tile1; ++tile) {
      const uint32_t i = tile * 32u + lane;
      if (i >= p.width) continue;
      const float x = __fadd_rn(p.x0, __fmul_rn((float)i, p.dx));
      float zr, zi, cr, ci;
      if (KIND == VRHI_ESCAPE_MANDELBROT) {
        zr = 0.f; zi = 0.f; cr = p.transposed ? y : x; ci = p.transposed ? x : y;
      } else {
        zr = p.transposed ? y : x; zi = p.transposed ? x : y; cr = p.cr; ci = p.ci;
      }
      uint32_t count = 0;
      float a = 0.f, b = 0.f;
      z_squares<MODE>(zr, zi, a, b);
      for (;;) {
        if (escaped<TEST>(z_norm2<MODE>(zr, zi, a, b), p.bound) || count >= p.max_iter) break;
        z_advance<MODE>(zr, zi, a, b, cr, ci);
        ++count;
      }
      store_count<OUT>(image, row_base + i, count, p.color_scale);
      if (wire) store_wire(wire, row_base + i, count);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Regrouping kernel (test "a+b > bound" with bound >= 4, |c| <= 1.5; MODE selects the exact or the
// contracted rounding sequence, the machinery is the same).
//
// Iteration counts inside a warp differ by orders of magnitude near the set, so one pixel per lane
// with a test on every step leaves most lanes idle (about 36 % lane efficiency on the 16384^2
// Julia workload).  This kernel keeps lanes busy and spends fewer instructions per step:
//
//  * FAST BLOCKS.  A lane runs U updates with no test and no counter: 6 instructions per step
//    (a=zr*zr, b=zi*zi, t=zr*zi, zi=fma(2,t,ci), a-b, +cr) for 8 algorithmic operations.  One test
//    at the end of the block decides whether the whole block was valid.  That is exact because,
//    for bound >= 4 and |c| <= 1.5, escape is monotonic even in binary32: once a+b > bound then
//    |z'| >= |z|^2 - |c| > 1.2|z|, so every later a+b is larger still, or Inf/NaN, and the test is
//    written !(s <= bound) so that NaN counts as escaped.  A lane whose block failed the test (or
//    would pass max_iter) is put back on its checkpoint and marked "finishing".
//  * CHECKED BLOCKS.  When at least T lanes are finishing or empty, the warp runs one block of U
//    steps with the test and the counter on every step; lanes still in flight simply advance,
//    finishing lanes find their exact count.  Finished pixels are stored and their lanes freed.
//  * POOL.  Freed lanes are refilled from a per-warp ring in shared memory.  The ring is fed by
//    INTAKE: 32 fresh pixels of a stolen tile run K checked steps in lock step (most pixels of the
//    far exterior end there and are stored coalesced); survivors are pushed to the ring with their
//    state.  Long-lived pixels therefore share warps with other long-lived pixels.
//  * WORK STEALING.  Warps pull batches of up to 16 tiles (512 pixels of one row) from a global
//    counter.  The host launches 4 CTAs per SM (2 for small images): the kernel is bound by
//    instruction issue, so the 6 CTAs the launch bounds allow bring nothing more.
//
// Nothing here waits on another warp or CTA: no spin loops, no barriers.
constexpr int kPoolCap = 64;

// U = steps per block, T = waiting lanes that trigger a checked block, K = checked steps a fresh pixel gets before it is pooled
template <int KIND, int OUT, int U, int T, int K = 8, int MODE = VRHI_ESCAPE_EXACT, bool WIRE = false>
__global__ void __launch_bounds__(256, 6) escape_regroup_kernel(EscapeDev p, void *image, uint32_t *work_counter, uint16_t *wire = nullptr) {
  constexpr bool PER_PIXEL_C = (KIND == VRHI_ESCAPE_MANDELBROT);
  __shared__ float s_zr[8][kPoolCap], s_zi[8][kPoolCap];
  __shared__ uint32_t s_idx[8][kPoolCap], s_cnt[8][kPoolCap];
  __shared__ float s_cr[PER_PIXEL_C ? 8 : 1][kPoolCap], s_ci[PER_PIXEL_C ? 8 : 1][kPoolCap];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  const uint32_t FULL = 0xffffffffu;
  float *pzr = s_zr[warp], *pzi = s_zi[warp];
  uint32_t *pidx = s_idx[warp], *pcnt = s_cnt[warp];
  float *pcr = s_cr[PER_PIXEL_C ? warp : 0], *pci = s_ci[PER_PIXEL_C ? warp : 0];
  // parameters live in registers: the hot loops must not go back to the constant bank
  const float bound = p.bound, x0 = p.x0, dx = p.dx, color_scale = p.color_scale;
  const uint32_t max_iter = p.max_iter, width = p.width;
  const bool transposed = p.transposed != 0;
  const uint32_t fast_limit = max_iter - (uint32_t)U;  // the host guarantees max_iter >= U: cnt <= fast_limit means a whole block fits

  // warp-uniform state
  uint32_t pool_head = 0, pool_tail = 0, pool_n = 0;
  bool fresh = true;
  uint32_t tile = 0, tile_end = 0, row_base = 0;
  float row_y = 0.f;
  // lane state (a = zr*zr and b = zi*zi ride along so that a step costs six instructions)
  float zr = 0.f, zi = 0.f, a = 0.f, b = 0.f, cr = p.cr, ci = p.ci;
  uint32_t cnt = 0, idx = 0;
  bool occ = false;  // the lane holds a pixel
  bool run = false;  // ... and that pixel may go through unchecked blocks (occ && !run: it is finishing)

  auto intake = [&]() {
    if (tile >= tile_end) {
      uint32_t batch = 0;
      if (lane == 0) batch = atomicAdd(work_counter, 1u);
      batch = __shfl_sync(FULL, batch, 0);
      if (batch >= p.n_batches) { fresh = false; return; }
      const uint32_t r = batch / p.batches_per_row;
      tile = (batch - r * p.batches_per_row) * p.batch_tiles;
      tile_end = min(tile + p.batch_tiles, p.tiles_per_row);
      const uint32_t j = owned_row_to_image_row(p, r);
      row_y = __fadd_rn(p.y0, __fmul_rn((float)j, p.dy));
      row_base = j * width;
    }
    const uint32_t i = tile * 32u + lane;
    ++tile;
    const bool valid = i < width;
    const float x = __fadd_rn(x0, __fmul_rn((float)i, dx));
    float fzr, fzi, fcr, fci;
    const float re = transposed ? row_y : x, im = transposed ? x : row_y;
    if (PER_PIXEL_C) { fzr = 0.f; fzi = 0.f; fcr = re; fci = im; }
    else { fzr = re; fzi = im; fcr = cr; fci = ci; }
    uint32_t fcnt = 0;
    bool flive = valid;
    float fa = 0.f, fb = 0.f;
    z_squares<MODE>(fzr, fzi, fa, fb);
    // K steps with a test on each; dead lanes keep computing (their values are never used), so the
    // loop body is straight-line code.  The host guarantees max_iter >= K: no cap test in here.
#pragma unroll
    for (int k = 0; k < K; ++k) {
      flive = flive && (z_norm2<MODE>(fzr, fzi, fa, fb) <= bound);
      // most tiles lie far outside the set and die within two or three steps, all lanes together
      if ((k == 2 || k == 4) && k < K - 1 && !__any_sync(FULL, flive)) break;
      z_advance<MODE>(fzr, fzi, fa, fb, fcr, fci);
      fcnt += flive ? 1u : 0u;
    }
    if (PER_PIXEL_C) {
      // pixels whose own constant is too large for the fast path are finished here, step by step
      bool slow = flive && !(fmaf(fcr, fcr, fci * fci) <= 2.25f);
      while (__any_sync(FULL, slow)) {
        if (slow) {
          if (!(z_norm2<MODE>(fzr, fzi, fa, fb) <= bound) || fcnt >= max_iter) { slow = false; flive = false; }
          else {
            z_advance<MODE>(fzr, fzi, fa, fb, fcr, fci);
            ++fcnt;
          }
        }
      }
    }
    if (valid && !flive) {
      store_count<OUT>(image, (size_t)(row_base + i), fcnt, color_scale);
      if (WIRE) store_wire(wire, (size_t)(row_base + i), fcnt);
    }
    const uint32_t m = __ballot_sync(FULL, flive);
    if (m) {
      if (flive) {
        const uint32_t slot = (pool_head + __popc(m & lt_mask)) & (kPoolCap - 1);
        pzr[slot] = fzr; pzi[slot] = fzi; pidx[slot] = row_base + i; pcnt[slot] = fcnt;
        if (PER_PIXEL_C) { pcr[slot] = fcr; pci[slot] = fci; }
      }
      const uint32_t n = __popc(m);
      pool_head = (pool_head + n) & (kPoolCap - 1);
      pool_n += n;
      __syncwarp();
    }
  };

  // One block of U steps with the test on every step, straight-line: a lane that has stopped
  // keeps computing values nobody reads, only its counter is frozen.  CAP = false is used when no
  // lane can reach max_iter inside the block, which saves the counter comparison on every step.
  auto checked_block = [&](auto cap_tag) {
    constexpr bool CAP = decltype(cap_tag)::value;
    z_squares<MODE>(zr, zi, a, b);  // finishing lanes were put back on their checkpoint: refresh the squares
    bool live = occ;
#pragma unroll
    for (int k = 0; k < U; ++k) {
      live = live && (z_norm2<MODE>(zr, zi, a, b) <= bound);
      if (CAP) live = live && (cnt < max_iter);
      z_advance<MODE>(zr, zi, a, b, cr, ci);
      cnt += live ? 1u : 0u;
    }
    // the block made U tests and up to U updates; a lane whose fast block failed only at its very
    // last state needs the test of that state too (tests are idempotent, so this changes nothing
    // for lanes that pass)
    live = live && (z_norm2<MODE>(zr, zi, a, b) <= bound);
    if (CAP) live = live && (cnt < max_iter);
    if (occ && !live) {
      store_count<OUT>(image, (size_t)idx, cnt, color_scale);
      if (WIRE) store_wire(wire, (size_t)idx, cnt);
    }
    occ = live;
    run = live;  // a finishing lane always ends inside the block
  };

  for (;;) {
    // ---- refill: feed the pool until every empty lane can be served, then hand out entries
    const uint32_t free_mask = __ballot_sync(FULL, !occ);
    if (free_mask) {
      const uint32_t need = __popc(free_mask);
      while (pool_n < need && fresh) intake();
      if (pool_n) {
        const uint32_t r = __popc(free_mask & lt_mask);
        if (!occ && r < pool_n) {
          const uint32_t slot = (pool_tail + r) & (kPoolCap - 1);
          zr = pzr[slot]; zi = pzi[slot]; idx = pidx[slot]; cnt = pcnt[slot];
          if (PER_PIXEL_C) { cr = pcr[slot]; ci = pci[slot]; }
          z_squares<MODE>(zr, zi, a, b);
          occ = true; run = true;
        }
        const uint32_t popped = min(need, pool_n);
        pool_tail = (pool_tail + popped) & (kPoolCap - 1);
        pool_n -= popped;
        __syncwarp();
      }
    }
    uint32_t waiting = __popc(__ballot_sync(FULL, !run));
    if (waiting == 32u && __ballot_sync(FULL, occ) == 0u) break;  // pool empty, no fresh tiles, no lane in flight
    // ---- fast blocks until enough lanes want attention (all of them once nothing can be refilled)
    const uint32_t threshold = (!fresh && pool_n == 0) ? 32u : (uint32_t)T;
    while (waiting < threshold) {
      const float ckr = zr, cki = zi;
#pragma unroll
      for (int k = 0; k < U; ++k) z_advance<MODE>(zr, zi, a, b, cr, ci);
      // lanes that are not running (empty or finishing) computed garbage: they, and lanes whose
      // block failed, go back to the checkpoint; a and b are refreshed by the checked block
      run = run && (z_norm2<MODE>(zr, zi, a, b) <= bound) && (cnt <= fast_limit);
      if (run) cnt += U;
      else { zr = ckr; zi = cki; }
      waiting = __popc(__ballot_sync(FULL, !run));
    }
    // ---- one checked block: finishing lanes find their exact count, the others just advance
    if (__any_sync(FULL, occ && cnt > fast_limit)) checked_block(std::true_type{});
    else checked_block(std::false_type{});
  }
}

template <int KIND, int MODE, int TEST>
static void launch_checked_out(int out, int grid, cudaStream_t s, const EscapeDev &p, void *image, uint32_t *ctr, uint16_t *wire) {
  switch (out) {
    case VRHI_OUT_COUNT_U32: escape_checked_kernel<KIND, MODE, TEST, VRHI_OUT_COUNT_U32><<<grid, 256, 0, s>>>(p, image, ctr, wire); break;
    case VRHI_OUT_COUNT_U16: escape_checked_kernel<KIND, MODE, TEST, VRHI_OUT_COUNT_U16><<<grid, 256, 0, s>>>(p, image, ctr, nullptr); break;
    default: escape_checked_kernel<KIND, MODE, TEST, VRHI_OUT_COLOR_F32><<<grid, 256, 0, s>>>(p, image, ctr, nullptr); break;
  }
}

template <int KIND, int MODE>
static void launch_checked_test(int test, int out, int grid, cudaStream_t s, const EscapeDev &p, void *image, uint32_t *ctr, uint16_t *wire) {
  if (test == VRHI_TEST_NORM2_GT)
    launch_checked_out<KIND, MODE, VRHI_TEST_NORM2_GT>(out, grid, s, p, image, ctr, wire);
  else
    launch_checked_out<KIND, MODE, VRHI_TEST_NORM_GE>(out, grid, s, p, image, ctr, wire);
}

int launch_escape_time(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_escape_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 1 && n_args != 2) return fail(VRHI_ERR_INVALID, "escape_time takes the image and, optionally, a uint16 wire copy; got %d arguments", n_args);
  if (!writable(args[0])) return fail(VRHI_ERR_INVALID, "escape_time: the image buffer is read-only (class %s)", vrhi_arg_class_name(args[0].buf_cls));
  uint16_t *wire = nullptr;
  if (n_args == 2) {
    if (q.output != VRHI_OUT_COUNT_U32) return fail(VRHI_ERR_INVALID, "escape_time: the uint16 wire copy goes with uint32 counts only");
    if (q.max_iter > 65535u) return fail(VRHI_ERR_UNSUPPORTED, "escape_time: a uint16 wire copy needs max_iter <= 65535");
    if (!writable(args[1])) return fail(VRHI_ERR_INVALID, "escape_time: the wire buffer is read-only (class %s)", vrhi_arg_class_name(args[1].buf_cls));
    if (args[1].bytes < (uint64_t)q.width * q.height * 2) return fail(VRHI_ERR_SIZE, "escape_time: the wire view holds %llu bytes, %llu needed", (unsigned long long)args[1].bytes, (unsigned long long)q.width * q.height * 2);
    wire = reinterpret_cast<uint16_t *>(args[1].ptr);
  }
  if (q.kind > VRHI_ESCAPE_JULIA || q.mode > VRHI_ESCAPE_FAST || q.test > VRHI_TEST_NORM_GE || q.output > VRHI_OUT_COLOR_F32)
    return fail(VRHI_ERR_INVALID, "escape_time: kind/mode/test/output out of range");
  if (q.width == 0 || q.height == 0) return fail(VRHI_ERR_SIZE, "escape_time: empty image");
  if (q.output == VRHI_OUT_COUNT_U16 && q.max_iter > 65535u) return fail(VRHI_ERR_UNSUPPORTED, "escape_time: uint16 counts need max_iter <= 65535");
  if (q.max_iter > (1u << 24) && q.output == VRHI_OUT_COLOR_F32) return fail(VRHI_ERR_UNSUPPORTED, "escape_time: colour output needs max_iter <= 2^24");
  const size_t elem = q.output == VRHI_OUT_COUNT_U16 ? 2 : 4;
  const uint64_t need = (uint64_t)q.width * q.height * elem;
  if (args[0].bytes < need) return fail(VRHI_ERR_SIZE, "escape_time: image view holds %llu bytes, %llu needed", (unsigned long long)args[0].bytes, (unsigned long long)need);

  EscapeDev p{};
  p.width = q.width; p.height = q.height; p.max_iter = q.max_iter;
  p.x0 = q.x0; p.y0 = q.y0; p.dx = q.dx; p.dy = q.dy; p.cr = q.cr; p.ci = q.ci;
  p.bound = q.bound; p.color_scale = q.color_scale;
  p.transposed = (q.flags & VRHI_ESCAPE_FLAG_TRANSPOSED) ? 1u : 0u;
  if (q.chunk_rows == 0) {
    p.chunk_rows = q.height; p.chunk_first = 0; p.chunk_step = 1; p.rows_owned = q.height;
  } else {
    if (q.chunk_step == 0) return fail(VRHI_ERR_INVALID, "escape_time: chunk_step must be >= 1");
    p.chunk_rows = q.chunk_rows; p.chunk_first = q.chunk_first; p.chunk_step = q.chunk_step;
    uint64_t rows = 0;
    for (uint32_t k = 0; k < q.chunk_count; ++k) {
      uint64_t c = (uint64_t)q.chunk_first + (uint64_t)k * q.chunk_step;
      uint64_t r0 = c * q.chunk_rows;
      if (r0 >= q.height) return fail(VRHI_ERR_SIZE, "escape_time: chunk %llu starts beyond the image", (unsigned long long)c);
      uint64_t r1 = r0 + q.chunk_rows;
      if (r1 > q.height) {
        if (k + 1 != q.chunk_count) return fail(VRHI_ERR_SIZE, "escape_time: only the last chunk may be short");
        r1 = q.height;
      }
      rows += r1 - r0;
    }
    p.rows_owned = (uint32_t)rows;
  }
  if (p.rows_owned == 0) return VRHI_OK;  // an empty band is not an error
  p.neg_zero = -0.0f;
  // tuning aids, read once per process
  static const int env_batch = [] { const char *e = getenv("VRHI_ESCAPE_BATCH"); return e ? atoi(e) : 0; }();
  static const int env_per_sm = [] { const char *e = getenv("VRHI_ESCAPE_CTAS_PER_SM"); return e ? atoi(e) : 0; }();
  static const int env_pair = [] { const char *e = getenv("VRHI_ESCAPE_PAIR"); return e ? atoi(e) : 1; }();  // 0: one pixel per lane
  const int sms = st->dev->prop.multiProcessorCount;
  // The regrouping kernels take what their exactness argument covers; everything else, and callers
  // that ask for it, runs the step-by-step kernel.
  const double c2 = (double)q.cr * q.cr + (double)q.ci * q.ci;
  const bool regroup_ok = q.test == VRHI_TEST_NORM2_GT && q.bound >= 4.0f && q.bound < 3.0e38f &&
                          q.max_iter >= 64u && q.max_iter <= (1u << 30) && (uint64_t)q.width * q.height <= 0xffffffffull &&
                          (q.kind == VRHI_ESCAPE_MANDELBROT || c2 <= 2.25) && !(q.flags & VRHI_ESCAPE_FLAG_CHECKED_ONLY);
  const bool pair = regroup_ok && env_pair != 0;
  const uint32_t tile_px = pair ? 64u : 32u;  // pixels a warp takes in per intake trip
  p.tiles_per_row = (q.width + tile_px - 1) / tile_px;
  {
    // batch = unit of work stealing: 512 pixels of one row for large images; small images get smaller
    // batches so that every resident warp still sees several of them and the tail stays short
    const uint64_t resident_warps = (uint64_t)sms * 48;
    const uint64_t tiles = (uint64_t)p.tiles_per_row * p.rows_owned;
    const uint64_t most = 512 / tile_px;
    uint64_t bt = tiles / (resident_warps * 8);
    const uint64_t least = pair ? 1 : 2;
    p.batch_tiles = (uint32_t)(bt < least ? least : bt > most ? most : bt);
    if (env_batch >= 1 && env_batch <= 64) p.batch_tiles = (uint32_t)env_batch;
  }
  p.batches_per_row = (p.tiles_per_row + p.batch_tiles - 1) / p.batch_tiles;
  uint64_t nb = (uint64_t)p.batches_per_row * p.rows_owned;
  if (nb > 0xfffffff0ull) return fail(VRHI_ERR_UNSUPPORTED, "escape_time: image too large for 32-bit batch indices");
  p.n_batches = (uint32_t)nb;

  uint64_t warps_needed = nb;
  int grid = (int)((warps_needed + 7) / 8 < (uint64_t)sms * 8 ? (warps_needed + 7) / 8 : (uint64_t)sms * 8);
  // A frame of a few batches per warp (the 640 x 320 frame of fractal.py:7-8 is one) is dealt out
  // statically: resetting a work counter would be a second node per frame and cost as much as the frame.
  const bool dealt = !regroup_ok && nb <= (uint64_t)grid * 8 * 4;
  uint32_t *counter = nullptr;
  if (!dealt) {
    uint32_t *ctrl = nullptr;
    VRHI_TRY(stream_arena(st, 0, &ctrl, nullptr));
    counter = ctrl + CTRL_WORK0;
    VRHI_CUDA(cudaMemsetAsync(counter, 0, sizeof(uint32_t), st->s));
  }
  if (regroup_ok) {
    // Measured on B200: 3-4 CTAs of 256 threads per SM are as fast as more (the kernels are bound by
    // issue or by the binary32 pipe, not by latency); small images run faster still with 2, because
    // each warp then owns enough tiles to keep its pool busy and the drain at the end is shorter.
    uint64_t ctas = (nb + 7) / 8;
    const uint64_t px_total = (uint64_t)p.tiles_per_row * tile_px * p.rows_owned;
    uint64_t per_sm = px_total / ((uint64_t)sms * 4 * 8) < 1024 ? 2 : 4;
    if (env_per_sm >= 1 && env_per_sm <= 6) per_sm = (uint64_t)env_per_sm;
    const uint64_t cap = (uint64_t)sms * per_sm;
    grid = (int)(ctas < cap ? ctas : cap);
    // Small images (2 blocks per SM) are short launches, usually frames of a sequence: there the next
    // frame's blocks should move in while this frame's last ones drain (65 -> 41 us per 1080p frame
    // with two alternating streams), and a few tens of microseconds cannot go far out of balance.
    const bool pin = per_sm >= 4;
    if (pair) {
      VRHI_TRY(launch_escape_pair(st, q, p, grid, (int)per_sm, pin, args[0].ptr, counter, wire));
      return post_launch(st, "escape_time (two pixels per lane)");
    }
    // U = 12, T = 8, K = 8: a sweep on B200 (U = 8..16, T = 4..12, K = 4..12) was flat within 2 % around this point
#define REGROUP(KIND, OUT)                                                                                             \
  do {                                                                                                                 \
    if (q.mode == VRHI_ESCAPE_EXACT) VRHI_TRY(launch_pinned(escape_regroup_kernel<KIND, OUT, 12, 8, 8, VRHI_ESCAPE_EXACT>, grid, (int)per_sm, st, p, args[0].ptr, counter, nullptr, pin)); \
    else VRHI_TRY(launch_pinned(escape_regroup_kernel<KIND, OUT, 12, 8, 8, VRHI_ESCAPE_FAST>, grid, (int)per_sm, st, p, args[0].ptr, counter, nullptr, pin));   \
  } while (0)
#define REGROUP_WIRE(KIND)                                                                                              \
  do {                                                                                                                 \
    if (q.mode == VRHI_ESCAPE_EXACT) VRHI_TRY(launch_pinned(escape_regroup_kernel<KIND, VRHI_OUT_COUNT_U32, 12, 8, 8, VRHI_ESCAPE_EXACT, true>, grid, (int)per_sm, st, p, args[0].ptr, counter, wire, pin)); \
    else VRHI_TRY(launch_pinned(escape_regroup_kernel<KIND, VRHI_OUT_COUNT_U32, 12, 8, 8, VRHI_ESCAPE_FAST, true>, grid, (int)per_sm, st, p, args[0].ptr, counter, wire, pin));   \
  } while (0)
    if (wire) {
      if (q.kind == VRHI_ESCAPE_MANDELBROT) REGROUP_WIRE(VRHI_ESCAPE_MANDELBROT);
      else REGROUP_WIRE(VRHI_ESCAPE_JULIA);
    } else if (q.kind == VRHI_ESCAPE_MANDELBROT) {
      if (q.output == VRHI_OUT_COUNT_U32) REGROUP(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COUNT_U32);
      else if (q.output == VRHI_OUT_COUNT_U16) REGROUP(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COUNT_U16);
      else REGROUP(VRHI_ESCAPE_MANDELBROT, VRHI_OUT_COLOR_F32);
    } else {
      if (q.output == VRHI_OUT_COUNT_U32) REGROUP(VRHI_ESCAPE_JULIA, VRHI_OUT_COUNT_U32);
      else if (q.output == VRHI_OUT_COUNT_U16) REGROUP(VRHI_ESCAPE_JULIA, VRHI_OUT_COUNT_U16);
      else REGROUP(VRHI_ESCAPE_JULIA, VRHI_OUT_COLOR_F32);
    }
#undef REGROUP
#undef REGROUP_WIRE
    return post_launch(st, "escape_time (regrouping)");
  }
  if (q.kind == VRHI_ESCAPE_MANDELBROT) {
    if (q.mode == VRHI_ESCAPE_EXACT) launch_checked_test<VRHI_ESCAPE_MANDELBROT, VRHI_ESCAPE_EXACT>(q.test, q.output, grid, st->s, p, args[0].ptr, counter, wire);
    else launch_checked_test<VRHI_ESCAPE_MANDELBROT, VRHI_ESCAPE_FAST>(q.test, q.output, grid, st->s, p, args[0].ptr, counter, wire);
  } else {
    if (q.mode == VRHI_ESCAPE_EXACT) launch_checked_test<VRHI_ESCAPE_JULIA, VRHI_ESCAPE_EXACT>(q.test, q.output, grid, st->s, p, args[0].ptr, counter, wire);
    else launch_checked_test<VRHI_ESCAPE_JULIA, VRHI_ESCAPE_FAST>(q.test, q.output, grid, st->s, p, args[0].ptr, counter, wire);
  }
  return post_launch(st, "escape_time");
}

// ---------------------------------------------------------------------------------------------
// FP32 issue-rate probe: independent FFMA chains, 8 per thread, nothing else in the loop body.
__global__ void __launch_bounds__(256) fp32_probe_kernel(float *out, uint64_t iters, float seed) {
  float v0 = seed + threadIdx.x, v1 = v0 + 1.f, v2 = v0 + 2.f, v3 = v0 + 3.f;
  float v4 = v0 + 4.f, v5 = v0 + 5.f, v6 = v0 + 6.f, v7 = v0 + 7.f;
  const float m = 0.999f, c = 0.001f;
  for (uint64_t k = 0; k < iters; ++k) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      v0 = fmaf(v0, m, c); v1 = fmaf(v1, m, c); v2 = fmaf(v2, m, c); v3 = fmaf(v3, m, c);
      v4 = fmaf(v4, m, c); v5 = fmaf(v5, m, c); v6 = fmaf(v6, m, c); v7 = fmaf(v7, m, c);
    }
  }
  float r = ((v0 + v1) + (v2 + v3)) + ((v4 + v5) + (v6 + v7));
  if (r == 12345.678f) out[0] = r;  // keeps the chains alive without memory traffic
}

int launch_fp32_probe(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_probe_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 1 || args[0].bytes < 4 || !writable(args[0])) return fail(VRHI_ERR_INVALID, "fp32_probe takes one writable argument of at least 4 bytes");
  const int sms = st->dev->prop.multiProcessorCount;
  uint64_t threads = q.threads ? q.threads : (uint64_t)sms * 2048;
  uint64_t blocks = (threads + 255) / 256;
  if (blocks == 0 || blocks > 0x7fffffffull) return fail(VRHI_ERR_SIZE, "fp32_probe: thread count out of range");
  uint64_t iters = q.ffma_per_thread / 64;  // 64 FFMAs per loop trip
  fp32_probe_kernel<<<(unsigned)blocks, 256, 0, st->s>>>(reinterpret_cast<float *>(args[0].ptr), iters, 1.0f);
  return post_launch(st, "fp32_probe");
}

}  // namespace vrhi
