// Shared pieces of the escape-time kernels (k_escape.cu: one pixel per lane; k_escape_pair.cu: two
// pixels per lane in packed binary32 pairs): the device-side parameter block, the step primitives
// of the two arithmetic modes, and the store helpers.  Loop rules follow fractal.py:11-25.
#pragma once

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "vrhi_internal.h"

namespace vrhi {

struct EscapeDev {
  uint32_t width, height, max_iter;
  float x0, y0, dx, dy, cr, ci, bound, color_scale;
  uint32_t chunk_rows, chunk_first, chunk_step;
  uint32_t rows_owned;       // rows this launch computes
  uint32_t tiles_per_row;    // ceil(width / tile), tile = 32 pixels (one per lane) or 64 (two per lane)
  uint32_t batch_tiles;      // tiles per stolen batch (a batch never straddles a row)
  uint32_t batches_per_row;
  uint32_t n_batches;
  uint32_t transposed;       // 1: the row coordinate is the real part and the column coordinate the imaginary part
  float neg_zero;            // -0.0f, set by the host: an addend the assembler cannot fold (k_escape_pair.cu)
  uint8_t *bytes;            // optional third copy of every count, min(count, 255), at the same pixel index (nullptr: none)
};

// Step primitives.  EXACT keeps a = zr*zr and b = zi*zi alongside z so that one update costs six
// instructions; FAST lets multiply-adds fuse (four instructions per update) and is a different,
// equally well-defined rounding sequence:
//     test  s = fma(zi, zi, zr*zr)        update  zi' = fma(zr+zr, zi, ci);  zr' = fma(zr, zr, fma(-zi, zi, cr))
template <int MODE>
__device__ __forceinline__ void z_squares(float zr, float zi, float &a, float &b) {
  if (MODE == VRHI_ESCAPE_EXACT) { a = __fmul_rn(zr, zr); b = __fmul_rn(zi, zi); }
}
template <int MODE>
__device__ __forceinline__ float z_norm2(float zr, float zi, float a, float b) {
  if (MODE == VRHI_ESCAPE_EXACT) return __fadd_rn(a, b);
  return __fmaf_rn(zi, zi, __fmul_rn(zr, zr));
}
template <int MODE>
__device__ __forceinline__ void z_advance(float &zr, float &zi, float &a, float &b, float cr, float ci) {
  if (MODE == VRHI_ESCAPE_EXACT) {
    const float t = __fmul_rn(zr, zi);
    zi = __fmaf_rn(2.0f, t, ci);
    zr = __fadd_rn(__fsub_rn(a, b), cr);
    a = __fmul_rn(zr, zr);
    b = __fmul_rn(zi, zi);
  } else {
    const float nzi = __fmaf_rn(__fadd_rn(zr, zr), zi, ci);
    zr = __fmaf_rn(zr, zr, __fmaf_rn(-zi, zi, cr));
    zi = nzi;
  }
}

template <int TEST>
__device__ __forceinline__ bool escaped(float s, float bound) {
  if (TEST == VRHI_TEST_NORM2_GT) return !(s <= bound);  // NaN counts as escaped; s > bound otherwise
  return !(__fsqrt_rn(s) < bound);
}

template <int OUT>
__device__ __forceinline__ void store_count(void *image, size_t pix, uint32_t count, float color_scale) {
  if (OUT == VRHI_OUT_COUNT_U32)
    static_cast<uint32_t *>(image)[pix] = count;
  else if (OUT == VRHI_OUT_COUNT_U16)
    static_cast<uint16_t *>(image)[pix] = (uint16_t)count;
  else
    static_cast<float *>(image)[pix] = __fsub_rn(1.0f, __fmul_rn((float)count, color_scale));
}

// Second copy of a count as uint16 at the same pixel index (the compact form a rank sends to its
// peers when the image is gathered; counts up to 65535 lose nothing).
// With `bytes` also min(count, 255) as one byte: the plane that crosses NVLink where the counts are squeezed
// (a byte of 255 tells the receiving side to fetch the uint16 count).
__device__ __forceinline__ void store_wire(uint16_t *wire, uint8_t *bytes, size_t pix, uint32_t count) {
  wire[pix] = (uint16_t)count;
  if (bytes) bytes[pix] = (uint8_t)min(count, 255u);
}

// A launch that its caller declared independent of the launches before it is started with the
// programmatic-serialization attribute: its blocks may become resident as soon as every block of the
// launch before it has passed begin_overlap(), i.e. at once, beside that launch's blocks.  Every
// block calls end_overlap() last: the grid then cannot complete before the grid before it has, so
// whatever follows on the stream in the ordinary way still finds everything earlier finished.
// Both are no-ops in a launch without the attribute and nothing after it that carries it.
__device__ __forceinline__ void begin_overlap() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void end_overlap() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch `kern` on the stream; `overlap`: with the attribute described above.
template <class Kern, class... Args>
cudaError_t launch_maybe_overlapped(Kern kern, int grid, int block, size_t dyn, cudaStream_t s, bool overlap, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = s;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = overlap ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Order in which a launch visits its rows: from the middle outwards (k = 0 is the middle row).  The
// expensive rows of these images lie around the middle and hold the pixels that run for thousands
// of steps; a pixel started late is a tail nothing else covers (one warp, one dependent chain, tens
// of microseconds), so those rows go first and the cheap outer rows, whose pixels end within a few
// steps, go last.
__device__ __forceinline__ uint32_t middle_out(uint32_t k, uint32_t rows) {
  const uint32_t mid = rows >> 1, h = (k + 1u) >> 1;
  // k odd: rows below the middle (mid-1, mid-2, ...); k even: the middle and above; past the shorter side the rest follows in order
  if (k & 1u) return h <= mid ? mid - h : k;
  return mid + h < rows ? mid + h : rows - 1u - k;
}

// Row of the image that owned row r maps to (rows are owned in chunks dealt round-robin).
__device__ __forceinline__ uint32_t owned_row_to_image_row(const EscapeDev &p, uint32_t r) {
  uint32_t k = r / p.chunk_rows;
  return (p.chunk_first + k * p.chunk_step) * p.chunk_rows + (r - k * p.chunk_rows);
}

// Launch of a work-stealing escape-time kernel with its residency pinned.  Such a kernel is a
// persistent grid of `per_sm` blocks per SM; that only balances if the blocks really sit per_sm to
// an SM.  On an idle GPU they do, but when blocks of another stream's kernel are resident at launch
// time the hardware packs the grid onto whichever SMs have room, and the SMs that got more than
// their share then finish late (measured: 3.7 ms instead of 2.5 ms for the 16384^2 image).  Unused
// dynamic shared memory sized so that exactly per_sm blocks fit makes the surplus blocks wait for
// their own SM instead.  `pin` false launches without the padding.
// The opt-in limit of a kernel is only ever raised, under the lock and per device, so concurrent
// launches from several host threads never see a limit below what they ask for.
template <class Kern>
int launch_pinned(Kern kern, int grid, int per_sm, vrhi_stream_t *st, const EscapeDev &p, void *image, uint32_t *counter,
                  uint16_t *wire, bool pin = true, bool overlap = false) {
  struct Entry { size_t fixed; size_t limit; };
  static std::mutex mu;
  static std::unordered_map<uint64_t, Entry> cache;  // key: kernel address mixed with the device ordinal
  static const int pin_env = [] { const char *e = getenv("VRHI_ESCAPE_PIN"); return e ? atoi(e) : 1; }();  // tuning aid: 0 = no padding
  const uint64_t key = (uint64_t)reinterpret_cast<uintptr_t>(reinterpret_cast<const void *>(kern)) * 64u + (uint64_t)st->dev->ordinal;
  size_t dyn = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
      cudaFuncAttributes fa{};
      VRHI_CUDA(cudaFuncGetAttributes(&fa, kern));
      it = cache.emplace(key, Entry{fa.sharedSizeBytes, 0}).first;
    }
    if (pin && pin_env != 0 && per_sm >= 1) {
      const size_t per_sm_bytes = st->dev->prop.sharedMemPerMultiprocessor;  // each resident block also reserves 1 KB
      size_t total = ((size_t)((double)per_sm_bytes / (per_sm + 0.5)) - 1024) & ~size_t(127);
      const size_t optin = st->dev->prop.sharedMemPerBlockOptin;
      if (total > optin) total = optin;
      dyn = total > it->second.fixed ? total - it->second.fixed : 0;
    }
    if (dyn > it->second.limit) {
      VRHI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
      it->second.limit = dyn;
    }
  }
  if (overlap) VRHI_CUDA(launch_maybe_overlapped(kern, grid, 256, dyn, st->s, true, p, image, counter, wire));
  else kern<<<grid, 256, dyn, st->s>>>(p, image, counter, wire);
  return VRHI_OK;
}

// the two-pixels-per-lane kernel (k_escape_pair.cu)
int launch_escape_pair(vrhi_stream_t *st, const vrhi_escape_params &q, const EscapeDev &p, int grid, int per_sm, bool pin, bool overlap,
                       void *image, uint32_t *counter, uint16_t *wire);

}  // namespace vrhi
