// Receiving side of the image gather: counts arrive from the peers as uint16 (half the bytes on
// NVLink) and are widened into the uint32 image here.
#include "vrhi_internal.h"

namespace vrhi {

// One block row of 256 threads widens 2048 pixels of one image row: a 16-byte load of eight
// counts, two 16-byte stores.  Rows are enumerated slab by slab over the chunks the skipped rank
// does not own.  HBM-bound: 2 B read + 4 B written per pixel.
template <bool VEC>
__global__ void __launch_bounds__(256) widen_rows_u16_kernel(const uint16_t *__restrict__ wire, uint32_t *__restrict__ image,
                                                             uint32_t width, uint32_t height, uint32_t chunk_rows, uint32_t world,
                                                             uint32_t skip_rank, uint32_t slab_first, uint32_t total_rows) {
  const uint32_t nq = skip_rank < world ? world - 1 : world;
  const uint32_t rows_per_slab = nq * chunk_rows;
  for (uint32_t u = blockIdx.y; u < total_rows; u += gridDim.y) {
    const uint32_t slab = u / rows_per_slab, rem = u - slab * rows_per_slab;
    const uint32_t qq = rem / chunk_rows, rr = rem - qq * chunk_rows;
    const uint32_t q = qq + (qq >= skip_rank ? 1u : 0u);
    const uint64_t row = ((uint64_t)(slab_first + slab) * world + q) * chunk_rows + rr;
    if (row >= height) continue;
    const size_t base = (size_t)row * width;
    if (VEC) {
      const uint32_t v = blockIdx.x * 256u + threadIdx.x;
      if (v * 8u < width) {
        const uint4 in = __ldcs(reinterpret_cast<const uint4 *>(wire + base) + v);
        uint4 lo, hi;
        lo.x = in.x & 0xffffu; lo.y = in.x >> 16; lo.z = in.y & 0xffffu; lo.w = in.y >> 16;
        hi.x = in.z & 0xffffu; hi.y = in.z >> 16; hi.z = in.w & 0xffffu; hi.w = in.w >> 16;
        uint4 *out = reinterpret_cast<uint4 *>(image + base) + 2 * (size_t)v;
        __stcs(out, lo);
        __stcs(out + 1, hi);
      }
    } else {
      for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < width; i += gridDim.x * 256u) image[base + i] = wire[base + i];
    }
  }
}

int launch_widen_rows_u16(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params, size_t params_size) {
  vrhi_widen_params q;
  VRHI_TRY(read_params(params, params_size, &q));
  if (n_args != 2) return fail(VRHI_ERR_INVALID, "widen_rows_u16 takes 2 arguments (wire, image), got %d", n_args);
  if (!writable(args[1])) return fail(VRHI_ERR_INVALID, "widen_rows_u16: the image buffer is read-only (class %s)", vrhi_arg_class_name(args[1].buf_cls));
  if (q.width == 0 || q.height == 0) return fail(VRHI_ERR_SIZE, "widen_rows_u16: empty image");
  if (q.chunk_rows == 0 || q.world == 0) return fail(VRHI_ERR_INVALID, "widen_rows_u16: chunk_rows and world must be >= 1");
  const uint64_t px = (uint64_t)q.width * q.height;
  if (args[0].bytes < px * 2) return fail(VRHI_ERR_SIZE, "widen_rows_u16: the wire view holds %llu bytes, %llu needed", (unsigned long long)args[0].bytes, (unsigned long long)(px * 2));
  if (args[1].bytes < px * 4) return fail(VRHI_ERR_SIZE, "widen_rows_u16: the image view holds %llu bytes, %llu needed", (unsigned long long)args[1].bytes, (unsigned long long)(px * 4));
  const uint64_t n_chunks = ((uint64_t)q.height + q.chunk_rows - 1) / q.chunk_rows;
  const uint64_t n_slabs = (n_chunks + q.world - 1) / q.world;
  if ((uint64_t)q.slab_first + q.slab_count > n_slabs) return fail(VRHI_ERR_SIZE, "widen_rows_u16: slabs %u..%llu lie beyond the image's %llu", q.slab_first, (unsigned long long)q.slab_first + q.slab_count, (unsigned long long)n_slabs);
  const uint32_t nq = q.skip_rank < q.world ? q.world - 1 : q.world;
  const uint64_t total_rows = (uint64_t)q.slab_count * nq * q.chunk_rows;
  if (total_rows == 0) return VRHI_OK;  // nothing to widen (one rank, or an empty slab range)
  if (total_rows > 0xffffffffull) return fail(VRHI_ERR_UNSUPPORTED, "widen_rows_u16: too many rows");
  const bool vec = q.width % 8 == 0 && ((uintptr_t)args[0].ptr % 16 == 0) && ((uintptr_t)args[1].ptr % 16 == 0);
  dim3 grid;
  grid.y = (unsigned)(total_rows < 32768 ? total_rows : 32768);
  if (vec) {
    grid.x = (q.width / 8 + 255) / 256;
    widen_rows_u16_kernel<true><<<grid, 256, 0, st->s>>>(reinterpret_cast<const uint16_t *>(args[0].ptr), reinterpret_cast<uint32_t *>(args[1].ptr),
                                                         q.width, q.height, q.chunk_rows, q.world, q.skip_rank, q.slab_first, (uint32_t)total_rows);
  } else {
    grid.x = (q.width + 255) / 256 < 64 ? (q.width + 255) / 256 : 64;
    widen_rows_u16_kernel<false><<<grid, 256, 0, st->s>>>(reinterpret_cast<const uint16_t *>(args[0].ptr), reinterpret_cast<uint32_t *>(args[1].ptr),
                                                          q.width, q.height, q.chunk_rows, q.world, q.skip_rank, q.slab_first, (uint32_t)total_rows);
  }
  return post_launch(st, "widen_rows_u16");
}

}  // namespace vrhi
