// Receiving side of the image gather: counts arrive from the peers as uint16 (half the bytes on
// NVLink) and are widened into the uint32 image here.
#include <cstdlib>

#include "vrhi_internal.h"

namespace vrhi {

// A block widens whole image rows, one after the other (grid-stride over the rows to do): every
// thread keeps kWidenInFlight 16-byte loads in flight and writes two 16-byte stores for each.  The grid is
// kWidenBlocksPerSm blocks per SM and no more: the kernel runs beside the escape-time launches of
// the following groups, and a grid that filled every thread slot (8 blocks of 256 per SM, as a
// first form did, on a high-priority stream) kept those launches off the SMs until it was through
// (measured at 8 ranks: the four groups of a step computed in 0.9 ms instead of 0.4 ms).
// Rows are enumerated slab by slab over the chunks the skipped rank does not own.  HBM-bound: 2 B
// read + 4 B written per pixel.  (A first form with one short-lived block per 2048 pixels reached
// 2.1 TB/s; at four and eight ranks the widening of 3/4 and 7/8 of the image was then the longest
// part of a step.)
constexpr int kWidenInFlight = 8;
constexpr int kWidenBlocksPerSm = 2;

template <bool VEC>
__global__ void __launch_bounds__(256) widen_rows_u16_kernel(const uint16_t *__restrict__ wire, uint32_t *__restrict__ image,
                                                             uint32_t width, uint32_t height, uint32_t chunk_rows, uint32_t world,
                                                             uint32_t skip_rank, uint32_t slab_first, uint32_t slab_stride, uint32_t total_rows,
                                                             const uint32_t *ok = nullptr) {
  // `ok` is the verdict of a bounded wait that ran before this kernel in the stream: 0 = it gave up, widen nothing
  if (ok && *reinterpret_cast<const volatile uint32_t *>(ok) == 0u) return;
  const uint32_t nq = skip_rank < world ? world - 1 : world;
  const uint32_t rows_per_slab = nq * chunk_rows;
  for (uint32_t u = blockIdx.x; u < total_rows; u += gridDim.x) {
    const uint32_t slab = u / rows_per_slab, rem = u - slab * rows_per_slab;
    const uint32_t qq = rem / chunk_rows, rr = rem - qq * chunk_rows;
    const uint32_t q = qq + (qq >= skip_rank ? 1u : 0u);
    const uint64_t row = ((uint64_t)(slab_first + slab * slab_stride) * world + q) * chunk_rows + rr;
    if (row >= height) continue;
    const size_t base = (size_t)row * width;
    if (VEC) {
      const uint32_t segs = width / 8u;
      const uint4 *src = reinterpret_cast<const uint4 *>(wire + base);
      uint4 *dst = reinterpret_cast<uint4 *>(image + base);
      for (uint32_t v0 = threadIdx.x; v0 < segs; v0 += 256u * kWidenInFlight) {
        uint4 in[kWidenInFlight];
#pragma unroll
        for (int j = 0; j < kWidenInFlight; ++j)
          if (v0 + j * 256u < segs) in[j] = __ldcs(src + v0 + j * 256u);
#pragma unroll
        for (int j = 0; j < kWidenInFlight; ++j) {
          const uint32_t v = v0 + j * 256u;
          if (v < segs) {
            __stcs(dst + 2 * (size_t)v, make_uint4(in[j].x & 0xffffu, in[j].x >> 16, in[j].y & 0xffffu, in[j].y >> 16));
            __stcs(dst + 2 * (size_t)v + 1, make_uint4(in[j].z & 0xffffu, in[j].z >> 16, in[j].w & 0xffffu, in[j].w >> 16));
          }
        }
      }
    } else {
      for (uint32_t i = threadIdx.x; i < width; i += 256u) image[base + i] = wire[base + i];
    }
  }
}

// wire -> image for the given slabs; `ok` (optional) guards the launch, see the kernel
int widen_rows_u16(vrhi_stream_t *st, const uint16_t *wire, uint32_t *image, const vrhi_widen_params &q, const uint32_t *ok) {
  if (q.width == 0 || q.height == 0) return fail(VRHI_ERR_SIZE, "widen_rows_u16: empty image");
  if (q.chunk_rows == 0 || q.world == 0) return fail(VRHI_ERR_INVALID, "widen_rows_u16: chunk_rows and world must be >= 1");
  const uint64_t n_chunks = ((uint64_t)q.height + q.chunk_rows - 1) / q.chunk_rows;
  const uint64_t n_slabs = (n_chunks + q.world - 1) / q.world;
  const uint32_t stride = q.slab_stride ? q.slab_stride : 1u;
  if (q.slab_count && (uint64_t)q.slab_first + (uint64_t)(q.slab_count - 1) * stride >= n_slabs)
    return fail(VRHI_ERR_SIZE, "widen_rows_u16: slabs %u + k*%u, k < %u, reach beyond the image's %llu", q.slab_first, stride, q.slab_count, (unsigned long long)n_slabs);
  const uint32_t nq = q.skip_rank < q.world ? q.world - 1 : q.world;
  const uint64_t total_rows = (uint64_t)q.slab_count * nq * q.chunk_rows;
  if (total_rows == 0) return VRHI_OK;  // nothing to widen (one rank, or an empty slab range)
  if (total_rows > 0xffffffffull) return fail(VRHI_ERR_UNSUPPORTED, "widen_rows_u16: too many rows");
  const bool vec = q.width % 8 == 0 && ((uintptr_t)wire % 16 == 0) && ((uintptr_t)image % 16 == 0);
  const uint64_t cap = (uint64_t)st->dev->prop.multiProcessorCount * kWidenBlocksPerSm;  // a persistent grid over the rows
  const unsigned grid = (unsigned)(total_rows < cap ? total_rows : cap);
  if (vec)
    widen_rows_u16_kernel<true><<<grid, 256, 0, st->s>>>(wire, image, q.width, q.height, q.chunk_rows, q.world, q.skip_rank, q.slab_first, stride, (uint32_t)total_rows, ok);
  else
    widen_rows_u16_kernel<false><<<grid, 256, 0, st->s>>>(wire, image, q.width, q.height, q.chunk_rows, q.world, q.skip_rank, q.slab_first, stride, (uint32_t)total_rows, ok);
  return post_launch(st, "widen_rows_u16");
}

int launch_widen_rows_u16(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_widen_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 2) return fail(VRHI_ERR_INVALID, "widen_rows_u16 takes 2 arguments (wire, image), got %d", n_args);
  if (!writable(args[1])) return fail(VRHI_ERR_INVALID, "widen_rows_u16: the image buffer is read-only (class %s)", vrhi_arg_class_name(args[1].buf_cls));
  const uint64_t px = (uint64_t)q.width * q.height;
  if (args[0].bytes < px * 2) return fail(VRHI_ERR_SIZE, "widen_rows_u16: the wire view holds %llu bytes, %llu needed", (unsigned long long)args[0].bytes, (unsigned long long)(px * 2));
  if (args[1].bytes < px * 4) return fail(VRHI_ERR_SIZE, "widen_rows_u16: the image view holds %llu bytes, %llu needed", (unsigned long long)args[1].bytes, (unsigned long long)(px * 4));
  return widen_rows_u16(st, reinterpret_cast<const uint16_t *>(args[0].ptr), reinterpret_cast<uint32_t *>(args[1].ptr), q, nullptr);
}

// ---------------------------------------------------------------------------------------------
// Pull form of the gather: each rank reads its peers' uint16 rows straight out of their memory
// over NVLink and writes them, widened, into its own image: transfer and widening are one kernel,
// nothing is staged, and all peers are read at the same time.  Readiness travels as sequence
// numbers: after computing a group of slabs a rank stores the group's number into its slot of
// every peer's flag array (signal kernel); the pull kernel of that group first waits, with a time
// limit, until every peer's slot has reached the number.  The waiting side only ever waits for a
// kernel that runs on ANOTHER GPU and that depends on nothing of the waiter's later work.
struct PeerPtrs {
  const uint16_t *wire[VRHI_GATHER_MAX_WORLD];  // indexed by rank; the caller's own entry is unused
};
struct PeerFlags {
  uint32_t *flags[VRHI_GATHER_MAX_WORLD];
};

__global__ void gather_signal_kernel(PeerFlags peers, uint32_t n_peers, uint32_t slot, uint32_t seq) {
  if (threadIdx.x < n_peers) {
    __threadfence_system();  // this rank's rows (written by earlier kernels of the stream) before the number
    *reinterpret_cast<volatile uint32_t *>(peers.flags[threadIdx.x] + slot) = seq;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The wait is a kernel of its own, one warp: a waiting kernel that held many thread slots could keep
// this rank's own signal kernel (which its peers are waiting for) off the SMs.  Lane q polls slot q
// of this rank's flag array; the verdict goes to `ok` for the copy kernel that follows in the stream.
__global__ void gather_wait_kernel(const uint32_t *flags, uint32_t world, uint32_t rank, uint32_t seq, uint64_t wait_ns,
                                   int32_t *status, uint32_t *ok) {
  bool mine = true;
  if (threadIdx.x < world && threadIdx.x != rank) {
    const volatile uint32_t *f = flags + threadIdx.x;
    const uint64_t t0 = global_ns();
    while ((int32_t)(*f - seq) < 0) {  // sequence numbers compare modulo 2^32
      if (global_ns() - t0 > wait_ns) { mine = false; break; }
      __nanosleep(500);
    }
  }
  const bool all = __all_sync(0xffffffffu, mine);
  if (threadIdx.x == 0) {
    if (!all) atomicCAS(status, 0, VRHI_ERR_TIMEOUT);
    *ok = all ? 1u : 0u;
    __threadfence();
  }
}

constexpr int kPullRows = 4;  // rows in flight per thread: 64 bytes of remote loads outstanding

__global__ void __launch_bounds__(256) gather_pull_u16_kernel(PeerPtrs peers, const uint32_t *ok, uint32_t *__restrict__ image,
                                                              uint32_t width, uint32_t height, uint32_t chunk_rows, uint32_t world,
                                                              uint32_t rank, uint32_t slab_first, uint32_t slab_stride, uint32_t total_rows) {
  if (*reinterpret_cast<const volatile uint32_t *>(ok) == 0u) return;  // the wait gave up: copy nothing; the host finds VRHI_ERR_TIMEOUT
  const uint32_t rows_per_slab = (world - 1) * chunk_rows;
  const uint32_t v = blockIdx.x * 256u + threadIdx.x;
  const bool col_ok = v * 8u < width;
  for (uint32_t u0 = blockIdx.y; u0 < total_rows; u0 += gridDim.y * kPullRows) {
    uint4 in[kPullRows];
    size_t base[kPullRows];
    bool ok[kPullRows];
#pragma unroll
    for (int k = 0; k < kPullRows; ++k) {
      const uint32_t u = u0 + (uint32_t)k * gridDim.y;
      ok[k] = false;
      if (u < total_rows && col_ok) {
        const uint32_t slab = u / rows_per_slab, rem = u - slab * rows_per_slab;
        const uint32_t qq = rem / chunk_rows, rr = rem - qq * chunk_rows;
        const uint32_t q = qq + (qq >= rank ? 1u : 0u);
        const uint64_t row = ((uint64_t)(slab_first + slab * slab_stride) * world + q) * chunk_rows + rr;
        if (row < height) {
          ok[k] = true;
          base[k] = (size_t)row * width;
          in[k] = __ldcg(reinterpret_cast<const uint4 *>(peers.wire[q] + base[k]) + v);  // L2 only: never a stale L1 line
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kPullRows; ++k) {
      if (ok[k]) {
        uint4 lo, hi;
        lo.x = in[k].x & 0xffffu; lo.y = in[k].x >> 16; lo.z = in[k].y & 0xffffu; lo.w = in[k].y >> 16;
        hi.x = in[k].z & 0xffffu; hi.y = in[k].z >> 16; hi.z = in[k].w & 0xffffu; hi.w = in[k].w >> 16;
        uint4 *out = reinterpret_cast<uint4 *>(image + base[k]) + 2 * (size_t)v;
        __stcs(out, lo);
        __stcs(out + 1, hi);
      }
    }
  }
}

static int read_gather(const void *params, size_t params_size, vrhi_gather_params *q) {
  VRHI_TRY(read_params(params, params_size, q));
  if (q->world < 2 || q->world > VRHI_GATHER_MAX_WORLD) return fail(VRHI_ERR_INVALID, "gather: world must be 2..%d, got %u", VRHI_GATHER_MAX_WORLD, q->world);
  if (q->rank >= q->world) return fail(VRHI_ERR_INVALID, "gather: rank %u outside world %u", q->rank, q->world);
  return VRHI_OK;
}

int launch_gather_signal(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_gather_params q;
  VRHI_TRY(read_gather(params, params_size, &q));
  if (n_args != (int)q.world - 1) return fail(VRHI_ERR_INVALID, "gather_signal takes the flag arrays of the %u peers, got %d arguments", q.world - 1, n_args);
  PeerFlags pf{};
  for (int k = 0; k < n_args; ++k) {
    if (args[k].bytes < (uint64_t)q.world * 4) return fail(VRHI_ERR_SIZE, "gather_signal: flag array %d holds %llu bytes, %u needed", k, (unsigned long long)args[k].bytes, q.world * 4);
    if (!writable(args[k])) return fail(VRHI_ERR_INVALID, "gather_signal: flag array %d is read-only", k);
    pf.flags[k] = reinterpret_cast<uint32_t *>(args[k].ptr);
  }
  gather_signal_kernel<<<1, 32, 0, st->s>>>(pf, (uint32_t)n_args, q.rank, q.seq);
  return post_launch(st, "gather_signal");
}

int launch_gather_pull_u16(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_gather_params q;
  VRHI_TRY(read_gather(params, params_size, &q));
  if (n_args != (int)q.world + 1) return fail(VRHI_ERR_INVALID, "gather_pull_u16 takes flags, image and the %u peers' wire images (%u arguments), got %d", q.world - 1, q.world + 1, n_args);
  if (q.width == 0 || q.height == 0 || q.chunk_rows == 0) return fail(VRHI_ERR_SIZE, "gather_pull_u16: empty image or chunk");
  if (q.width % 8 != 0) return fail(VRHI_ERR_UNSUPPORTED, "gather_pull_u16: the width must be a multiple of 8 pixels (16-byte loads)");
  const uint64_t px = (uint64_t)q.width * q.height;
  if (args[0].bytes < (uint64_t)q.world * 4) return fail(VRHI_ERR_SIZE, "gather_pull_u16: the flag array is too small");
  if (!writable(args[1])) return fail(VRHI_ERR_INVALID, "gather_pull_u16: the image buffer is read-only (class %s)", vrhi_arg_class_name(args[1].buf_cls));
  if (args[1].bytes < px * 4) return fail(VRHI_ERR_SIZE, "gather_pull_u16: the image view holds %llu bytes, %llu needed", (unsigned long long)args[1].bytes, (unsigned long long)(px * 4));
  PeerPtrs pp{};
  int k = 2;
  for (uint32_t r = 0; r < q.world; ++r) {
    if (r == q.rank) continue;
    if (args[k].bytes < px * 2) return fail(VRHI_ERR_SIZE, "gather_pull_u16: the wire image of rank %u holds %llu bytes, %llu needed", r, (unsigned long long)args[k].bytes, (unsigned long long)(px * 2));
    if ((uintptr_t)args[k].ptr % 16) return fail(VRHI_ERR_INVALID, "gather_pull_u16: the wire image of rank %u is not 16-byte aligned", r);
    pp.wire[r] = reinterpret_cast<const uint16_t *>(args[k].ptr);
    ++k;
  }
  if ((uintptr_t)args[1].ptr % 16) return fail(VRHI_ERR_INVALID, "gather_pull_u16: the image is not 16-byte aligned");
  const uint64_t n_chunks = ((uint64_t)q.height + q.chunk_rows - 1) / q.chunk_rows;
  const uint64_t n_slabs = (n_chunks + q.world - 1) / q.world;
  const uint32_t stride = q.slab_stride ? q.slab_stride : 1u;
  if (q.slab_count && (uint64_t)q.slab_first + (uint64_t)(q.slab_count - 1) * stride >= n_slabs) return fail(VRHI_ERR_SIZE, "gather_pull_u16: slabs beyond the image");
  const uint64_t total_rows = (uint64_t)q.slab_count * (q.world - 1) * q.chunk_rows;
  if (total_rows == 0) return VRHI_OK;
  if (total_rows > 0xffffffffull) return fail(VRHI_ERR_UNSUPPORTED, "gather_pull_u16: too many rows");
  uint32_t *ctrl = nullptr;
  VRHI_TRY(stream_arena(st, 0, &ctrl, nullptr));
  dim3 grid;
  grid.x = (q.width / 8 + 255) / 256;
  // enough blocks to keep ~64 bytes x 256 threads x 4 blocks per SM of remote loads in flight, no more
  const uint64_t want_y = ((uint64_t)st->dev->prop.multiProcessorCount * 4 + grid.x - 1) / grid.x;
  const uint64_t max_y = (total_rows + kPullRows - 1) / kPullRows;
  grid.y = (unsigned)(want_y < max_y ? want_y : max_y);
  const uint64_t wait_ns = (uint64_t)(q.wait_ms ? q.wait_ms : 2000u) * 1000000ull;
  gather_wait_kernel<<<1, 32, 0, st->s>>>(reinterpret_cast<const uint32_t *>(args[0].ptr), q.world, q.rank, q.seq, wait_ns,
                                          reinterpret_cast<int32_t *>(ctrl + CTRL_STATUS), ctrl + CTRL_WAIT_OK);
  gather_pull_u16_kernel<<<grid, 256, 0, st->s>>>(pp, ctrl + CTRL_WAIT_OK, reinterpret_cast<uint32_t *>(args[1].ptr),
                                                  q.width, q.height, q.chunk_rows, q.world, q.rank, q.slab_first, stride, (uint32_t)total_rows);
  return post_launch(st, "gather_pull_u16", 2);
}

// ---------------------------------------------------------------------------------------------
// Push form of the gather, the one vrhi_exchange_* uses: after computing a group of slabs a rank
// copies its own uint16 rows out of its wire image into the same rows of every peer's wire image
// with plain 16-byte stores over NVLink (one load, world-1 stores per thread and trip), then raises
// its sequence number in every peer's flag array (gather_signal_kernel).  The kernel is built to
// run BESIDE the escape-time kernel of the next group: blocks of 128 threads and few registers, so
// that they fit into what four resident escape-time blocks leave of an SM, and a demand of a few
// bytes per clock and SM, which the issue slots that kernel leaves free cover.
struct PeerWires {
  uint16_t *wire[VRHI_GATHER_MAX_WORLD];  // the world-1 peers, any order
};

constexpr int kPushRows = 4;  // rows in flight per thread

__global__ void __launch_bounds__(128) gather_push_u16_kernel(PeerWires peers, uint32_t n_peers, const uint16_t *__restrict__ wire, uint32_t width,
                                                              uint32_t height, uint32_t chunk_rows, uint32_t world, uint32_t rank,
                                                              uint32_t slab_first, uint32_t slab_stride, uint32_t total_rows) {
  const uint32_t v = blockIdx.x * 128u + threadIdx.x;
  if (v * 8u >= width) return;
  for (uint32_t u0 = blockIdx.y; u0 < total_rows; u0 += gridDim.y * kPushRows) {
    uint4 in[kPushRows];
    size_t at[kPushRows];
    bool ok[kPushRows];
#pragma unroll
    for (int k = 0; k < kPushRows; ++k) {
      const uint32_t u = u0 + (uint32_t)k * gridDim.y;
      ok[k] = false;
      if (u < total_rows) {
        const uint32_t slab = u / chunk_rows, rr = u - slab * chunk_rows;
        const uint64_t row = ((uint64_t)(slab_first + slab * slab_stride) * world + rank) * chunk_rows + rr;
        if (row < height) {
          ok[k] = true;
          at[k] = (size_t)row * width / 8 + v;
          in[k] = __ldcg(reinterpret_cast<const uint4 *>(wire) + at[k]);  // written by the escape-time kernel just before: L2
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kPushRows; ++k)
      if (ok[k])
        for (uint32_t q = 0; q < n_peers; ++q) __stcg(reinterpret_cast<uint4 *>(peers.wire[q]) + at[k], in[k]);
  }
}

int gather_push_u16(vrhi_stream_t *st, uint16_t *const *peer_wires, uint32_t n_peers, const uint16_t *wire, const vrhi_gather_params &q) {
  if (n_peers == 0 || n_peers >= VRHI_GATHER_MAX_WORLD) return fail(VRHI_ERR_INVALID, "gather push: 1..%d peers", VRHI_GATHER_MAX_WORLD - 1);
  if (q.width % 8 != 0) return fail(VRHI_ERR_UNSUPPORTED, "gather push: the width must be a multiple of 8 pixels (16-byte accesses)");
  const uint32_t stride = q.slab_stride ? q.slab_stride : 1u;
  const uint64_t total_rows = (uint64_t)q.slab_count * q.chunk_rows;
  if (total_rows == 0) return VRHI_OK;
  if (total_rows > 0xffffffffull) return fail(VRHI_ERR_UNSUPPORTED, "gather push: too many rows");
  PeerWires pw{};
  for (uint32_t k = 0; k < n_peers; ++k) pw.wire[k] = peer_wires[k];
  dim3 grid;
  grid.x = (q.width / 8 + 127) / 128;
  // a few small blocks per SM: enough stores in flight for the link, little enough to sit beside another kernel
  static const int per_sm = [] { const char *e = getenv("VRHI_PUSH_BLOCKS_PER_SM"); const int v = e ? atoi(e) : 0; return v >= 1 && v <= 16 ? v : 2; }();  // tuning aid
  const uint64_t want_y = ((uint64_t)st->dev->prop.multiProcessorCount * per_sm + grid.x - 1) / grid.x;
  const uint64_t max_y = (total_rows + kPushRows - 1) / kPushRows;
  grid.y = (unsigned)(want_y < max_y ? want_y : max_y);
  gather_push_u16_kernel<<<grid, 128, 0, st->s>>>(pw, n_peers, wire, q.width, q.height, q.chunk_rows, q.world, q.rank, q.slab_first, stride, (uint32_t)total_rows);
  return post_launch(st, "gather_push_u16");
}

// ---------------------------------------------------------------------------------------------
// The counts squeezed to one byte where that loses nothing.  Far from the set almost every count is
// small (on the 16384^2 Julia image 97 % are below 255).  The escape-time kernel therefore writes,
// beside the uint32 image and the uint16 wire image, a plane of bytes min(count, 255) (its optional
// third argument); the copy engines move a rank's rows of that plane to the peers, half the bytes of
// the uint16 rows, and the receiving kernel below takes every 16-pixel granule from the byte plane
// unless the granule shows a byte of 255: then it fetches the granule's uint16 counts from the
// OWNER's wire image with two 16-byte loads over NVLink (6 % of the granules of that image).  No
// sending kernel, no lists, no counters, no capacity to overflow: an image of nothing but large
// counts costs 1.5 times the plain uint16 transfer, the usual image a little over half of it.
// The owner's wire image of a step stays untouched until two steps later (two images alternate),
// and a rank cannot run two steps ahead of a peer whose rows it needs: what is fetched is this step's.
struct OwnerWires {
  const uint16_t *wire[VRHI_GATHER_MAX_WORLD];  // every rank's uint16 wire image of this step, by rank (the caller's own is unused)
};

__device__ __forceinline__ bool has_ff(uint32_t w) { return __vcmpeq4(w, 0xffffffffu) != 0u; }

// Byte plane -> uint32 image.  Rows and blocks as in widen_rows_u16_kernel; a granule is 16 pixels.
__global__ void __launch_bounds__(256) widen_rows_squeezed_kernel(const uint8_t *__restrict__ bytes, OwnerWires owners,
                                                                  uint32_t *__restrict__ image, uint32_t width, uint32_t height,
                                                                  uint32_t chunk_rows, uint32_t world, uint32_t skip_rank, uint32_t slab_first,
                                                                  uint32_t slab_stride, uint32_t total_rows, const uint32_t *ok) {
  if (ok && *reinterpret_cast<const volatile uint32_t *>(ok) == 0u) return;
  const uint32_t nq = skip_rank < world ? world - 1 : world;
  const uint32_t rows_per_slab = nq * chunk_rows;
  const uint32_t segs = width / 16u;
  for (uint32_t u = blockIdx.x; u < total_rows; u += gridDim.x) {
    const uint32_t slab = u / rows_per_slab, rem = u - slab * rows_per_slab;
    const uint32_t qq = rem / chunk_rows, rr = rem - qq * chunk_rows;
    const uint32_t q = qq + (qq >= skip_rank ? 1u : 0u);
    const uint64_t row = ((uint64_t)(slab_first + slab * slab_stride) * world + q) * chunk_rows + rr;
    if (row >= height) continue;
    const size_t g0 = (size_t)row * segs;
    for (uint32_t v0 = threadIdx.x; v0 < segs; v0 += 256u * kWidenInFlight) {
      uint4 in[kWidenInFlight];
#pragma unroll
      for (int j = 0; j < kWidenInFlight; ++j)
        if (v0 + j * 256u < segs) in[j] = __ldcs(reinterpret_cast<const uint4 *>(bytes) + g0 + v0 + j * 256u);
#pragma unroll
      for (int j = 0; j < kWidenInFlight; ++j) {
        const uint32_t v = v0 + j * 256u;
        if (v >= segs) continue;
        const size_t at = g0 + v;
        const uint4 sq = in[j];
        uint4 *out = reinterpret_cast<uint4 *>(image) + 4 * at;
        if (has_ff(sq.x) || has_ff(sq.y) || has_ff(sq.z) || has_ff(sq.w)) {
          const uint4 *src = reinterpret_cast<const uint4 *>(owners.wire[q]) + 2 * at;   // rank q computed this row
          const uint4 a = __ldcg(src), b = __ldcg(src + 1);                                 // L2 only: never a stale L1 line
          __stcs(out, make_uint4(a.x & 0xffffu, a.x >> 16, a.y & 0xffffu, a.y >> 16));
          __stcs(out + 1, make_uint4(a.z & 0xffffu, a.z >> 16, a.w & 0xffffu, a.w >> 16));
          __stcs(out + 2, make_uint4(b.x & 0xffffu, b.x >> 16, b.y & 0xffffu, b.y >> 16));
          __stcs(out + 3, make_uint4(b.z & 0xffffu, b.z >> 16, b.w & 0xffffu, b.w >> 16));
        } else {
          __stcs(out, make_uint4(sq.x & 0xffu, (sq.x >> 8) & 0xffu, (sq.x >> 16) & 0xffu, sq.x >> 24));
          __stcs(out + 1, make_uint4(sq.y & 0xffu, (sq.y >> 8) & 0xffu, (sq.y >> 16) & 0xffu, sq.y >> 24));
          __stcs(out + 2, make_uint4(sq.z & 0xffu, (sq.z >> 8) & 0xffu, (sq.z >> 16) & 0xffu, sq.z >> 24));
          __stcs(out + 3, make_uint4(sq.w & 0xffu, (sq.w >> 8) & 0xffu, (sq.w >> 16) & 0xffu, sq.w >> 24));
        }
      }
    }
  }
}

int widen_rows_squeezed(vrhi_stream_t *st, const uint8_t *bytes, const uint16_t *const *wire_by_rank, uint32_t *image, const vrhi_widen_params &q, const uint32_t *ok) {
  if (q.world > VRHI_GATHER_MAX_WORLD) return fail(VRHI_ERR_INVALID, "widen (squeezed): at most %d ranks", VRHI_GATHER_MAX_WORLD);
  OwnerWires ow{};
  for (uint32_t r = 0; r < q.world; ++r) ow.wire[r] = wire_by_rank[r];
  if (q.width % 16 != 0) return fail(VRHI_ERR_UNSUPPORTED, "widen (squeezed): the width must be a multiple of 16 pixels");
  const uint32_t stride = q.slab_stride ? q.slab_stride : 1u;
  const uint32_t nq = q.skip_rank < q.world ? q.world - 1 : q.world;
  const uint64_t total_rows = (uint64_t)q.slab_count * nq * q.chunk_rows;
  if (total_rows == 0) return VRHI_OK;
  if (total_rows > 0xffffffffull) return fail(VRHI_ERR_UNSUPPORTED, "widen: too many rows");
  const uint64_t cap = (uint64_t)st->dev->prop.multiProcessorCount * kWidenBlocksPerSm;
  const unsigned grid = (unsigned)(total_rows < cap ? total_rows : cap);
  widen_rows_squeezed_kernel<<<grid, 256, 0, st->s>>>(bytes, ow, image, q.width, q.height, q.chunk_rows, q.world, q.skip_rank, q.slab_first, stride, (uint32_t)total_rows, ok);
  return post_launch(st, "widen_rows_squeezed");
}

int launch_widen_rows_u8(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_widen_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (q.world == 0 || q.world > VRHI_GATHER_MAX_WORLD) return fail(VRHI_ERR_INVALID, "widen_rows_u8: world must be 1..%d, got %u", VRHI_GATHER_MAX_WORLD, q.world);
  if (n_args != (int)q.world + 2) return fail(VRHI_ERR_INVALID, "widen_rows_u8 takes the byte plane, the image and the %u ranks' wire images (%u arguments), got %d", q.world, q.world + 2, n_args);
  if (!writable(args[1])) return fail(VRHI_ERR_INVALID, "widen_rows_u8: the image buffer is read-only (class %s)", vrhi_arg_class_name(args[1].buf_cls));
  if (q.width == 0 || q.height == 0 || q.chunk_rows == 0) return fail(VRHI_ERR_SIZE, "widen_rows_u8: empty image or chunk");
  const uint64_t px = (uint64_t)q.width * q.height;
  if (args[0].bytes < px) return fail(VRHI_ERR_SIZE, "widen_rows_u8: the byte plane holds %llu bytes, %llu needed", (unsigned long long)args[0].bytes, (unsigned long long)px);
  if (args[1].bytes < px * 4) return fail(VRHI_ERR_SIZE, "widen_rows_u8: the image view holds %llu bytes, %llu needed", (unsigned long long)args[1].bytes, (unsigned long long)(px * 4));
  const uint16_t *by_rank[VRHI_GATHER_MAX_WORLD] = {};
  for (uint32_t r = 0; r < q.world; ++r) {
    if (args[2 + r].bytes < px * 2) return fail(VRHI_ERR_SIZE, "widen_rows_u8: the wire image of rank %u holds %llu bytes, %llu needed", r, (unsigned long long)args[2 + r].bytes, (unsigned long long)(px * 2));
    by_rank[r] = reinterpret_cast<const uint16_t *>(args[2 + r].ptr);
  }
  const uint64_t n_chunks = ((uint64_t)q.height + q.chunk_rows - 1) / q.chunk_rows;
  const uint64_t n_slabs = (n_chunks + q.world - 1) / q.world;
  const uint32_t stride = q.slab_stride ? q.slab_stride : 1u;
  if (q.slab_count && (uint64_t)q.slab_first + (uint64_t)(q.slab_count - 1) * stride >= n_slabs) return fail(VRHI_ERR_SIZE, "widen_rows_u8: slabs beyond the image");
  return widen_rows_squeezed(st, reinterpret_cast<const uint8_t *>(args[0].ptr), by_rank, reinterpret_cast<uint32_t *>(args[1].ptr), q, nullptr);
}

// stores `seq` into slot `slot` of each of the n flag arrays (the peers')
int gather_signal(vrhi_stream_t *st, uint32_t *const *peer_flags, uint32_t n, uint32_t slot, uint32_t seq) {
  if (n == 0 || n >= VRHI_GATHER_MAX_WORLD) return fail(VRHI_ERR_INVALID, "gather signal: 1..%d peers", VRHI_GATHER_MAX_WORLD - 1);
  PeerFlags pf{};
  for (uint32_t k = 0; k < n; ++k) pf.flags[k] = peer_flags[k];
  gather_signal_kernel<<<1, 32, 0, st->s>>>(pf, n, slot, seq);
  return post_launch(st, "gather_signal");
}

// bounded wait until every peer's slot of `flags` has reached `seq`; the verdict lands in the stream's
// control block (CTRL_WAIT_OK, returned through *ok) for the kernel that follows
int gather_wait(vrhi_stream_t *st, const uint32_t *flags, uint32_t world, uint32_t rank, uint32_t seq, uint32_t wait_ms, const uint32_t **ok) {
  uint32_t *ctrl = nullptr;
  VRHI_TRY(stream_arena(st, 0, &ctrl, nullptr));
  const uint64_t wait_ns = (uint64_t)(wait_ms ? wait_ms : 2000u) * 1000000ull;
  gather_wait_kernel<<<1, 32, 0, st->s>>>(flags, world, rank, seq, wait_ns, reinterpret_cast<int32_t *>(ctrl + CTRL_STATUS), ctrl + CTRL_WAIT_OK);
  if (ok) *ok = ctrl + CTRL_WAIT_OK;
  return post_launch(st, "gather_wait");
}

// ---------------------------------------------------------------------------------------------
// Sum of small float arrays over the ranks (db and the loss of a row-sharded backward, reduction
// partials): every rank stores its n values into its own slot of every rank's mailbox (its own
// included), raises its sequence number, waits (bounded) for the others and adds the `world` slots
// in rank order: the same bits on every rank, no atomics.
struct PeerBoxes {
  float *box[VRHI_GATHER_MAX_WORLD];  // mailbox of every rank, indexed by rank: [world][capacity] floats
};

__global__ void __launch_bounds__(256) box_scatter_kernel(PeerBoxes boxes, uint32_t world, uint32_t rank, const float *__restrict__ src, uint32_t n, uint32_t capacity) {
  for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < n; i += gridDim.x * 256u) {
    const float v = src[i];
    for (uint32_t q = 0; q < world; ++q) __stcg(boxes.box[q] + (size_t)rank * capacity + i, v);
  }
}

__global__ void __launch_bounds__(256) box_sum_kernel(const float *box, const uint32_t *ok, uint32_t world, float *__restrict__ dst, uint32_t n, uint32_t capacity) {
  if (*reinterpret_cast<const volatile uint32_t *>(ok) == 0u) return;  // the wait gave up: leave dst alone; the host finds VRHI_ERR_TIMEOUT
  for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < n; i += gridDim.x * 256u) {
    float s = __ldcg(box + i);
    for (uint32_t q = 1; q < world; ++q) s = __fadd_rn(s, __ldcg(box + (size_t)q * capacity + i));
    dst[i] = s;
  }
}

int box_scatter(vrhi_stream_t *st, float *const *boxes, uint32_t world, uint32_t rank, const float *src, uint32_t n, uint32_t capacity) {
  PeerBoxes pb{};
  for (uint32_t k = 0; k < world; ++k) pb.box[k] = boxes[k];
  const unsigned blocks = (n + 255) / 256 < 64 ? (n + 255) / 256 : 64;
  box_scatter_kernel<<<blocks, 256, 0, st->s>>>(pb, world, rank, src, n, capacity);
  return post_launch(st, "all_reduce (scatter)");
}

int box_sum(vrhi_stream_t *st, const float *box, const uint32_t *ok, uint32_t world, float *dst, uint32_t n, uint32_t capacity) {
  const unsigned blocks = (n + 255) / 256 < 64 ? (n + 255) / 256 : 64;
  box_sum_kernel<<<blocks, 256, 0, st->s>>>(box, ok, world, dst, n, capacity);
  return post_launch(st, "all_reduce (sum)");
}

}  // namespace vrhi
