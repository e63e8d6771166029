// Multi-GPU half of libvrhi.so: groups of ranks (one process or thread per GPU of one box), the
// gather of an escape-time image whose row chunks were computed by different ranks, and the sum
// of small float arrays over the ranks.  The reference runs on one device (fractal.py:5), so
// nothing here has a counterpart there; see include/vrhi.h for the contract.
//
// No collective library is involved.  Ranks map each other's buffers (CUDA IPC between
// processes, peer access inside one process), move data with plain stores over NVLink from small
// kernels, and tell each other what has arrived through sequence numbers in flag arrays; every
// device-side wait is one warp with a time limit that records VRHI_ERR_TIMEOUT instead of hanging.
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "vrhi_internal.h"

using namespace vrhi;

namespace {

constexpr uint32_t kBoxCapacity = 16384;  // floats per rank and mailbox: the largest all-reduce
constexpr uint32_t kMaxWorld = VRHI_GATHER_MAX_WORLD;

struct ShareRecord {  // what a rank tells the others about one allocation
  int64_t pid;
  int32_t ordinal;
  int32_t pad;
  uint64_t ptr;
  cudaIpcMemHandle_t handle;
};

}  // namespace

struct vrhi_group_t {
  vrhi_device_t *dev;
  uint32_t world, rank;
  vrhi_allgather_fn allgather;
  void *user;
  std::vector<void *> opened;  // IPC mappings to close
  // small all-reduce: two mailboxes [world][kBoxCapacity] alternate from call to call
  float *box[2];
  float *all_box[2][kMaxWorld];    // every rank's mailbox, indexed by rank (own included)
  uint32_t *flags;                 // own flag array [world]
  uint32_t *peer_flags[kMaxWorld]; // the world-1 peers'
  uint32_t reduce_seq;
  uint32_t wait_ms;
  bool ready;  // creation got as far as the ranks' first meeting: destruction meets again
};

constexpr uint32_t kMaxPending = 16;
struct Pending {  // a published group whose transfer has not been enqueued yet
  uint32_t slab_first, slab_count, stride, seq;
};

struct vrhi_exchange_t {
  vrhi_group_t *grp;
  vrhi_buffer_t *image;
  uint32_t width, height, chunk_rows, n_slabs;
  vrhi_buffer_t *wire[2];               // own wire images (uint16 [height][width]); two alternate from step to step
  uint16_t *peer_wire[2][kMaxWorld];    // the world-1 peers', starting with rank+1
  // squeezed transfer (see k_gather.cu): counts cross as bytes, granules with large counts are fetched in full
  bool squeeze;
  vrhi_buffer_t *bytes[2];              // own byte planes [height][width], alternating like the wire images
  uint8_t *peer_bytes[2][kMaxWorld];    // the world-1 peers', starting with rank+1
  const uint16_t *wire_by_rank[2][kMaxWorld];  // every rank's wire images, indexed by rank
  uint32_t *flags;                      // own flag array [world]
  uint32_t *peer_flags[kMaxWorld];
  vrhi_stream_t *push[kMaxWorld], *arrive;  // internal streams: one per peer for the transfers to it; waits and widening
  uint32_t n_push;
  cudaEvent_t ev_push[kMaxWorld], ev_arrive;
  uint32_t cur, seq;
  uint64_t steps;
  Pending pending[kMaxPending];
  cudaEvent_t ev_group[kMaxPending];    // the point of the compute stream each pending group was published at
  uint32_t n_pending;
  std::vector<void *> *opened;          // IPC mappings of the peers' wire images and flags
  bool ready;
  // VRHI_EXCHANGE_TRACE=1: timed events behind each group's transfer and widening, printed by vrhi_exchange_check
  bool trace;
  uint32_t n_marks;                     // publishes of the current step
  cudaEvent_t t_computed[16], t_pushed[16], t_widened[16], t_done;
  uint32_t last_marks;
};

namespace {

int set_dev(vrhi_device_t *dev) {
  VRHI_CUDA(cudaSetDevice(dev->ordinal));
  return VRHI_OK;
}

// Make `local` (a cudaMalloc allocation of this rank) reachable by every rank and collect the
// pointers under which this rank reaches everybody else's; by_rank[own rank] = local.  Mappings
// of other processes' memory are noted in `opened`: they must be closed before the owner frees.
int share(vrhi_group_t *g, void *local, void **by_rank, std::vector<void *> *opened) {
  ShareRecord mine{};
  mine.pid = (int64_t)getpid();
  mine.ordinal = g->dev->ordinal;
  mine.ptr = (uint64_t)(uintptr_t)local;
  VRHI_CUDA(cudaIpcGetMemHandle(&mine.handle, local));
  std::vector<ShareRecord> all(g->world);
  if (g->world > 1) {
    int rc = g->allgather(g->user, &mine, all.data(), sizeof(ShareRecord));
    if (rc != 0) return fail(VRHI_ERR_PEER, "the caller's all-gather returned %d", rc);
  } else {
    all[0] = mine;
  }
  if (all[g->rank].pid != mine.pid || all[g->rank].ptr != mine.ptr)
    return fail(VRHI_ERR_PEER, "the caller's all-gather did not return this rank's record in slot %u", g->rank);
  for (uint32_t r = 0; r < g->world; ++r) {
    if (r == g->rank) { by_rank[r] = local; continue; }
    if (all[r].pid == mine.pid) {
      // another thread of this process: plain peer access
      if (all[r].ordinal != g->dev->ordinal) {
        cudaError_t e = cudaDeviceEnablePeerAccess(all[r].ordinal, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
        else if (e != cudaSuccess) return fail(VRHI_ERR_PEER, "no peer access from device %d to device %d: %s", g->dev->ordinal, all[r].ordinal, cudaGetErrorString(e));
      }
      by_rank[r] = (void *)(uintptr_t)all[r].ptr;
    } else {
      void *p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, all[r].handle, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(VRHI_ERR_PEER, "mapping rank %u's memory failed: %s", r, cudaGetErrorString(e));
      }
      opened->push_back(p);
      by_rank[r] = p;
    }
  }
  return VRHI_OK;
}

// How a rank's uint16 rows reach its peers where the counts are not squeezed: by the copy engines
// (default: they move the data without occupying SMs; measured at two ranks on the 16384^2 Julia
// image, 1.39 ms per step against 1.48 ms) or, with VRHI_PUSH_COPY_ENGINE=0, by a small storing
// kernel beside the next group's compute (kept for comparison).
bool use_copy_engines() {
  static const bool v = [] { const char *e = getenv("VRHI_PUSH_COPY_ENGINE"); return !e || atoi(e) != 0; }();
  return v;
}

// Whether the counts cross NVLink squeezed to bytes (see k_gather.cu): half the bytes for the copy engines
// to move, one more store per pixel for the escape-time kernel.  On by default from three ranks on,
// where the transfer is as long as the arithmetic or longer (at eight ranks each GPU takes in 7/8 of
// the image every step); VRHI_EXCHANGE_SQUEEZE=0/1 overrides.
bool use_squeeze(uint32_t world, uint32_t width) {
  static const int v = env_int("VRHI_EXCHANGE_SQUEEZE", 0, 1, -1);
  if (width % 16) return false;
  return v < 0 ? world >= 3 : v == 1;
}

// Ranks meet here: one round of the caller's all-gather.
int meet(vrhi_group_t *g) {
  if (g->world == 1) return VRHI_OK;
  uint32_t token = g->rank;
  std::vector<uint32_t> tokens(g->world);
  if (g->allgather(g->user, &token, tokens.data(), sizeof token) != 0) return fail(VRHI_ERR_PEER, "the caller's all-gather failed");
  return VRHI_OK;
}

// high_priority: blocks of the stream go first when an SM has room (the one-warp flag kernels behind the
// transfers); the widening kernels run at normal priority, behind the escape-time launches they share the GPU with
int make_stream(vrhi_device_t *dev, vrhi_stream_t **out, bool high_priority) {
  int lo = 0, hi = 0;
  VRHI_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  cudaStream_t s;
  VRHI_CUDA(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, high_priority ? hi : lo));
  vrhi_stream_t *st = new (std::nothrow) vrhi_stream_t{dev, s, true, nullptr, 0, 0};
  if (!st) {
    cudaStreamDestroy(s);
    return fail(VRHI_ERR_OOM, "host allocation failed");
  }
  *out = st;
  return VRHI_OK;
}

}  // namespace

extern "C" {

int vrhi_group_create(vrhi_device dev, uint32_t world, uint32_t rank, vrhi_allgather_fn allgather, void *user, vrhi_group *out_group) {
  if (!dev || !out_group) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_group = nullptr;
  if (world == 0 || world > kMaxWorld || rank >= world) return fail(VRHI_ERR_INVALID, "rank %u / world %u: a group has 1..%u ranks", rank, world, kMaxWorld);
  if (world > 1 && !allgather) return fail(VRHI_ERR_INVALID, "a group of more than one rank needs the caller's all-gather");
  VRHI_TRY(set_dev(dev));
  vrhi_group_t *g = new (std::nothrow) vrhi_group_t();
  if (!g) return fail(VRHI_ERR_OOM, "host allocation failed");
  g->dev = dev; g->world = world; g->rank = rank; g->allgather = allgather; g->user = user;
  g->reduce_seq = 0; g->wait_ms = 2000;
  g->box[0] = g->box[1] = nullptr; g->flags = nullptr;
  int rc = VRHI_OK;
  auto cleanup = [&](int code) { vrhi_group_destroy(g); return code; };
  for (int b = 0; b < 2 && rc == VRHI_OK; ++b) {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)world * kBoxCapacity * sizeof(float));
    if (e != cudaSuccess) { (void)cudaGetLastError(); return cleanup(fail(VRHI_ERR_OOM, "cudaMalloc of the group's mailbox failed: %s", cudaGetErrorString(e))); }
    g->box[b] = static_cast<float *>(p);
  }
  {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, 2u << 20);  // an allocation of its own (IPC maps whole allocations); `world` words are used
    if (e != cudaSuccess) { (void)cudaGetLastError(); return cleanup(fail(VRHI_ERR_OOM, "cudaMalloc of the group's flags failed: %s", cudaGetErrorString(e))); }
    g->flags = static_cast<uint32_t *>(p);
    e = cudaMemset(p, 0, 2u << 20);
    if (e != cudaSuccess) return cleanup(fail(VRHI_ERR_CUDA, "cudaMemset failed: %s", cudaGetErrorString(e)));
  }
  void *by_rank[kMaxWorld];
  for (int b = 0; b < 2; ++b) {
    rc = share(g, g->box[b], by_rank, &g->opened);
    if (rc != VRHI_OK) return cleanup(rc);
    for (uint32_t r = 0; r < world; ++r) g->all_box[b][r] = static_cast<float *>(by_rank[r]);
  }
  rc = share(g, g->flags, by_rank, &g->opened);
  if (rc != VRHI_OK) return cleanup(rc);
  for (uint32_t k = 0, r = 0; r < world; ++r)
    if (r != rank) g->peer_flags[k++] = static_cast<uint32_t *>(by_rank[r]);
  // every rank has zeroed its flags before anybody raises one
  g->ready = true;
  rc = meet(g);
  if (rc != VRHI_OK) return cleanup(rc);
  *out_group = g;
  return VRHI_OK;
}

int vrhi_group_destroy(vrhi_group g) {
  if (!g) return VRHI_OK;
  cudaSetDevice(g->dev->ordinal);
  cudaDeviceSynchronize();
  for (void *p : g->opened) cudaIpcCloseMemHandle(p);
  // a rank's memory must outlive every other rank's mapping of it: meet once all mappings are closed
  int rc = g->ready ? meet(g) : VRHI_OK;
  for (int b = 0; b < 2; ++b)
    if (g->box[b]) cudaFree(g->box[b]);
  if (g->flags) cudaFree(g->flags);
  delete g;
  return rc;
}

int vrhi_group_info(vrhi_group g, uint32_t *out_world, uint32_t *out_rank) {
  if (!g) return fail(VRHI_ERR_INVALID, "NULL group");
  if (out_world) *out_world = g->world;
  if (out_rank) *out_rank = g->rank;
  return VRHI_OK;
}

int vrhi_group_set_wait_ms(vrhi_group g, uint32_t wait_ms) {
  if (!g) return fail(VRHI_ERR_INVALID, "NULL group");
  g->wait_ms = wait_ms ? wait_ms : 2000;
  return VRHI_OK;
}

int vrhi_group_all_reduce_sum_f32(vrhi_group g, vrhi_buffer buf, uint64_t offset, uint64_t n, vrhi_stream stream) {
  if (!g || !buf || !stream) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (buf->dev != g->dev || stream->dev != g->dev) return fail(VRHI_ERR_INVALID, "buffer and stream must live on the group's device");
  stream->escape_chain = 0;
  if (offset % 4) return fail(VRHI_ERR_SIZE, "offset %llu is not a multiple of 4", (unsigned long long)offset);
  if (n > kBoxCapacity) return fail(VRHI_ERR_SIZE, "all-reduce of %llu floats: at most %u per call", (unsigned long long)n, kBoxCapacity);
  if (offset > buf->bytes || n * 4 > buf->bytes - offset) return fail(VRHI_ERR_SIZE, "range exceeds the buffer");
  if (buf->cls == VRHI_INPUT || buf->cls == VRHI_UNIFORM || buf->cls == VRHI_UNIFORM_CONSTANT) return fail(VRHI_ERR_INVALID, "the buffer is read-only (class %s)", vrhi_arg_class_name(buf->cls));
  if (n == 0 || g->world == 1) return VRHI_OK;
  VRHI_TRY(set_dev(g->dev));
  float *data = reinterpret_cast<float *>(static_cast<char *>(buf->ptr) + offset);
  const uint32_t seq = ++g->reduce_seq;
  const int b = (int)(seq & 1u);
  VRHI_TRY(box_scatter(stream, g->all_box[b], g->world, g->rank, data, (uint32_t)n, kBoxCapacity));
  VRHI_TRY(gather_signal(stream, g->peer_flags, g->world - 1, g->rank, seq));
  const uint32_t *ok = nullptr;
  VRHI_TRY(gather_wait(stream, g->flags, g->world, g->rank, seq, g->wait_ms, &ok));
  VRHI_TRY(box_sum(stream, g->box[b], ok, g->world, data, (uint32_t)n, kBoxCapacity));
  return VRHI_OK;
}

/* ------------------------------------------------------------------ image exchange ------ */

int vrhi_exchange_create(vrhi_group g, vrhi_buffer image, uint32_t width, uint32_t height, uint32_t chunk_rows, vrhi_exchange *out_ex) {
  if (!g || !image || !out_ex) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_ex = nullptr;
  if (image->dev != g->dev) return fail(VRHI_ERR_INVALID, "the image lives on another device than the group");
  if (width == 0 || height == 0 || chunk_rows == 0) return fail(VRHI_ERR_SIZE, "empty image or chunk");
  if (width % 8) return fail(VRHI_ERR_UNSUPPORTED, "the exchange needs a width that is a multiple of 8 pixels (16-byte accesses)");
  const uint64_t px = (uint64_t)width * height;
  if (image->bytes < px * 4) return fail(VRHI_ERR_SIZE, "the image holds %llu bytes, %llu needed", (unsigned long long)image->bytes, (unsigned long long)(px * 4));
  if (image->cls == VRHI_INPUT || image->cls == VRHI_UNIFORM || image->cls == VRHI_UNIFORM_CONSTANT) return fail(VRHI_ERR_INVALID, "the image is read-only (class %s)", vrhi_arg_class_name(image->cls));
  const uint64_t n_chunks = ((uint64_t)height + chunk_rows - 1) / chunk_rows;
  if (height % chunk_rows || n_chunks % g->world) return fail(VRHI_ERR_UNSUPPORTED, "the exchange needs chunks that divide the image evenly over the ranks (%llu chunks of %u rows, %u ranks)", (unsigned long long)n_chunks, chunk_rows, g->world);
  VRHI_TRY(set_dev(g->dev));
  vrhi_exchange_t *ex = new (std::nothrow) vrhi_exchange_t();
  if (!ex) return fail(VRHI_ERR_OOM, "host allocation failed");
  memset(static_cast<void *>(ex), 0, sizeof *ex);
  ex->grp = g; ex->image = image; ex->width = width; ex->height = height; ex->chunk_rows = chunk_rows;
  ex->n_slabs = (uint32_t)(n_chunks / g->world);
  ex->opened = new (std::nothrow) std::vector<void *>();
  if (!ex->opened) { delete ex; return fail(VRHI_ERR_OOM, "host allocation failed"); }
  auto cleanup = [&](int code) { vrhi_exchange_destroy(ex); return code; };
  for (int b = 0; b < 2; ++b) {
    int rc = vrhi_buffer_create(g->dev, px * 2, VRHI_IMAGE, &ex->wire[b]);
    if (rc != VRHI_OK) return cleanup(rc);
  }
  {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, 2u << 20);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return cleanup(fail(VRHI_ERR_OOM, "cudaMalloc of the exchange's flags failed: %s", cudaGetErrorString(e))); }
    ex->flags = static_cast<uint32_t *>(p);
    if (cudaMemset(p, 0, 2u << 20) != cudaSuccess) return cleanup(fail(VRHI_ERR_CUDA, "cudaMemset failed"));
  }
  ex->squeeze = g->world > 1 && use_squeeze(g->world, width);
  ex->trace = g->world > 1 && env_int("VRHI_EXCHANGE_TRACE", 0, 1, 0) == 1;
  if (ex->trace) {
    cudaEventCreate(&ex->t_done);
    for (int k = 0; k < 16; ++k) { cudaEventCreate(&ex->t_computed[k]); cudaEventCreate(&ex->t_pushed[k]); cudaEventCreate(&ex->t_widened[k]); }
  }
  void *by_rank[kMaxWorld];
  for (int b = 0; b < 2 && ex->squeeze; ++b) {
    int rc = vrhi_buffer_create(g->dev, px, VRHI_IMAGE, &ex->bytes[b]);
    if (rc != VRHI_OK) return cleanup(rc);
    rc = share(g, ex->bytes[b]->ptr, by_rank, ex->opened);
    if (rc != VRHI_OK) return cleanup(rc);
    for (uint32_t k = 0; k + 1 < g->world; ++k) ex->peer_bytes[b][k] = static_cast<uint8_t *>(by_rank[(g->rank + 1 + k) % g->world]);
  }
  for (int b = 0; b < 2; ++b) {
    int rc = share(g, ex->wire[b]->ptr, by_rank, ex->opened);
    if (rc != VRHI_OK) return cleanup(rc);
    // start with the next rank so that, at any moment, the ranks store to different peers
    for (uint32_t k = 0; k + 1 < g->world; ++k) ex->peer_wire[b][k] = static_cast<uint16_t *>(by_rank[(g->rank + 1 + k) % g->world]);
    for (uint32_t r = 0; r < g->world; ++r) ex->wire_by_rank[b][r] = static_cast<const uint16_t *>(by_rank[r]);
  }
  {
    int rc = share(g, ex->flags, by_rank, ex->opened);
    if (rc != VRHI_OK) return cleanup(rc);
    for (uint32_t k = 0; k + 1 < g->world; ++k) ex->peer_flags[k] = static_cast<uint32_t *>(by_rank[(g->rank + 1 + k) % g->world]);
  }
  // copy engines: a stream per peer, so that the transfers to different peers run on different engines at once;
  // the storing kernel serves all peers from one launch and needs one stream
  // One stream carries the copies to all peers, one after the other (every rank starts with its next neighbour, so at
  // any moment the ranks send to different peers).  A stream per peer (VRHI_PUSH_STREAMS=0) measured the same at four
  // ranks and costs three times the driver calls.
  static const bool per_peer = env_int("VRHI_PUSH_STREAMS", 0, 1, 1) == 0;  // comparison aid
  ex->n_push = per_peer && g->world > 2 ? g->world - 1 : 1;
  int rc = VRHI_OK;
  for (uint32_t k = 0; k < ex->n_push && rc == VRHI_OK; ++k) rc = make_stream(g->dev, &ex->push[k], true);
  if (rc == VRHI_OK) rc = make_stream(g->dev, &ex->arrive, false);
  if (rc != VRHI_OK) return cleanup(rc);
  uint32_t *ctrl = nullptr;
  rc = stream_arena(ex->arrive, 0, &ctrl, nullptr);  // the waits' status word: allocate now, not inside a step
  if (rc != VRHI_OK) return cleanup(rc);
  if (cudaEventCreateWithFlags(&ex->ev_arrive, cudaEventDisableTiming) != cudaSuccess)
    return cleanup(fail(VRHI_ERR_CUDA, "cudaEventCreate failed"));
  for (uint32_t k = 0; k < ex->n_push; ++k)
    if (cudaEventCreateWithFlags(&ex->ev_push[k], cudaEventDisableTiming) != cudaSuccess) return cleanup(fail(VRHI_ERR_CUDA, "cudaEventCreate failed"));
  for (uint32_t k = 0; k < kMaxPending; ++k)
    if (cudaEventCreateWithFlags(&ex->ev_group[k], cudaEventDisableTiming) != cudaSuccess) return cleanup(fail(VRHI_ERR_CUDA, "cudaEventCreate failed"));
  if (cudaDeviceSynchronize() != cudaSuccess) return cleanup(fail(VRHI_ERR_CUDA, "cudaDeviceSynchronize failed"));
  ex->ready = true;
  rc = meet(g);  // every rank has zeroed its flags before anybody raises one
  if (rc != VRHI_OK) return cleanup(rc);
  *out_ex = ex;
  return VRHI_OK;
}

int vrhi_exchange_destroy(vrhi_exchange ex) {
  if (!ex) return VRHI_OK;
  cudaSetDevice(ex->grp->dev->ordinal);
  cudaDeviceSynchronize();
  for (uint32_t k = 0; k < kMaxWorld; ++k)
    if (ex->push[k]) vrhi_stream_destroy(ex->push[k]);
  if (ex->arrive) vrhi_stream_destroy(ex->arrive);
  for (uint32_t k = 0; k < kMaxWorld; ++k)
    if (ex->ev_push[k]) cudaEventDestroy(ex->ev_push[k]);
  for (uint32_t k = 0; k < kMaxPending; ++k)
    if (ex->ev_group[k]) cudaEventDestroy(ex->ev_group[k]);
  if (ex->ev_arrive) cudaEventDestroy(ex->ev_arrive);
  if (ex->trace) {
    cudaEventDestroy(ex->t_done);
    for (int k = 0; k < 16; ++k) { cudaEventDestroy(ex->t_computed[k]); cudaEventDestroy(ex->t_pushed[k]); cudaEventDestroy(ex->t_widened[k]); }
  }
  if (ex->opened)
    for (void *p : *ex->opened) cudaIpcCloseMemHandle(p);
  delete ex->opened;
  // a rank's wire images must outlive every other rank's mapping of them
  int rc = ex->ready ? meet(ex->grp) : VRHI_OK;
  for (int b = 0; b < 2; ++b) vrhi_buffer_destroy(ex->wire[b]);
  for (int b = 0; b < 2; ++b) vrhi_buffer_destroy(ex->bytes[b]);
  if (ex->flags) cudaFree(ex->flags);
  delete ex;
  return rc;
}

int vrhi_exchange_planes(vrhi_exchange ex, vrhi_buffer *out_wire, vrhi_buffer *out_bytes) {
  if (!ex || !out_wire || !out_bytes) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_wire = ex->wire[ex->cur];
  *out_bytes = ex->squeeze ? ex->bytes[ex->cur] : nullptr;
  return VRHI_OK;
}

}  // extern "C" (reopened below)

namespace {

// Enqueue the transfer and the arrival of every group published since the last flush, in order.
int flush_pending(vrhi_exchange_t *ex) {
  vrhi_group_t *g = ex->grp;
  for (uint32_t i = 0; i < ex->n_pending; ++i) {
    const Pending &pd = ex->pending[i];
    const uint32_t slab_first = pd.slab_first, slab_count = pd.slab_count, stride = pd.stride, seq = pd.seq;
    cudaEvent_t ev = ex->ev_group[i];
    const bool mark = ex->trace && ex->n_marks < 16;
    // sending side, behind the launches that computed these slabs
    for (uint32_t k = 0; k < ex->n_push; ++k) VRHI_CUDA(cudaStreamWaitEvent(ex->push[k]->s, ev, 0));
    if (ex->squeeze || use_copy_engines()) {
      // the rank's rows by the copy engines, one strided copy per peer, and the peers' flags behind them.  Squeezing:
      // rows of the byte plane (the receiving side fetches what a byte cannot hold from this rank's uint16 wire image)
      const uint64_t elem = ex->squeeze ? 1 : 2;
      const uint64_t chunk_bytes = (uint64_t)ex->chunk_rows * ex->width * elem;
      const uint64_t offset = ((uint64_t)slab_first * g->world + g->rank) * chunk_bytes, pitch = (uint64_t)g->world * stride * chunk_bytes;
      const char *src = static_cast<const char *>(ex->squeeze ? ex->bytes[ex->cur]->ptr : ex->wire[ex->cur]->ptr) + offset;
      for (uint32_t k = 0; k + 1 < g->world; ++k) {
        vrhi_stream_t *ps = ex->push[ex->n_push > 1 ? k : 0];
        char *dst = (ex->squeeze ? reinterpret_cast<char *>(ex->peer_bytes[ex->cur][k]) : reinterpret_cast<char *>(ex->peer_wire[ex->cur][k])) + offset;
        VRHI_CUDA(cudaMemcpy2DAsync(dst, pitch, src, pitch, chunk_bytes, slab_count, cudaMemcpyDeviceToDevice, ps->s));
        if (ex->n_push > 1) VRHI_TRY(gather_signal(ps, &ex->peer_flags[k], 1, g->rank, seq));
      }
      if (ex->n_push == 1) VRHI_TRY(gather_signal(ex->push[0], ex->peer_flags, g->world - 1, g->rank, seq));
    } else {
      vrhi_gather_params q{};
      q.size = sizeof q; q.width = ex->width; q.height = ex->height; q.chunk_rows = ex->chunk_rows; q.world = g->world; q.rank = g->rank;
      q.slab_first = slab_first; q.slab_count = slab_count; q.slab_stride = stride; q.seq = seq; q.wait_ms = g->wait_ms;
      VRHI_TRY(gather_push_u16(ex->push[0], ex->peer_wire[ex->cur], g->world - 1, static_cast<const uint16_t *>(ex->wire[ex->cur]->ptr), q));
      VRHI_TRY(gather_signal(ex->push[0], ex->peer_flags, g->world - 1, g->rank, seq));
    }
    if (mark) VRHI_CUDA(cudaEventRecord(ex->t_pushed[ex->n_marks], ex->push[ex->n_push - 1]->s));
    // receiving side: when every peer's rows of this group have landed, widen them into the image; ordered
    // behind the caller's stream as well, so that what it enqueued before the publish (a download of the
    // previous step's image, say) is done with the image before a fast peer's rows are widened into it
    VRHI_CUDA(cudaStreamWaitEvent(ex->arrive->s, ev, 0));
    const uint32_t *ok = nullptr;
    VRHI_TRY(gather_wait(ex->arrive, ex->flags, g->world, g->rank, seq, g->wait_ms, &ok));
    vrhi_widen_params w{};
    w.size = sizeof w; w.width = ex->width; w.height = ex->height; w.chunk_rows = ex->chunk_rows; w.world = g->world; w.skip_rank = g->rank;
    w.slab_first = slab_first; w.slab_count = slab_count; w.slab_stride = stride;
    if (ex->squeeze) VRHI_TRY(widen_rows_squeezed(ex->arrive, static_cast<const uint8_t *>(ex->bytes[ex->cur]->ptr), ex->wire_by_rank[ex->cur], static_cast<uint32_t *>(ex->image->ptr), w, ok));
    else VRHI_TRY(widen_rows_u16(ex->arrive, static_cast<const uint16_t *>(ex->wire[ex->cur]->ptr), static_cast<uint32_t *>(ex->image->ptr), w, ok));
    if (mark) VRHI_CUDA(cudaEventRecord(ex->t_widened[ex->n_marks++], ex->arrive->s));
  }
  ex->n_pending = 0;
  return VRHI_OK;
}

}  // namespace

extern "C" {

int vrhi_exchange_publish(vrhi_exchange ex, vrhi_stream compute, uint32_t slab_first, uint32_t slab_count, uint32_t slab_stride) {
  if (!ex || !compute) return fail(VRHI_ERR_INVALID, "NULL argument");
  vrhi_group_t *g = ex->grp;
  if (compute->dev != g->dev) return fail(VRHI_ERR_INVALID, "the stream belongs to another device than the group");
  compute->escape_chain = 0;
  const uint32_t stride = slab_stride ? slab_stride : 1u;
  if (slab_count == 0) return fail(VRHI_ERR_SIZE, "an empty group of slabs cannot be published (every rank must publish the same groups)");
  if ((uint64_t)slab_first + (uint64_t)(slab_count - 1) * stride >= ex->n_slabs) return fail(VRHI_ERR_SIZE, "slabs %u + k*%u, k < %u, reach beyond the image's %u", slab_first, stride, slab_count, ex->n_slabs);
  if (g->world == 1) return VRHI_OK;
  VRHI_TRY(set_dev(g->dev));
  // Only the point of the compute stream is recorded here, so that the caller's next launch is not held
  // up by the dozen driver calls a group's transfer takes (with seven peers they cost more host time than a
  // group of an eighth of the image takes to compute); the transfer itself is enqueued by the next call that
  // is not a publish (complete, check, destroy), or when kMaxPending groups have gathered.
  if (ex->n_pending == kMaxPending) VRHI_TRY(flush_pending(ex));
  Pending &pd = ex->pending[ex->n_pending];
  VRHI_CUDA(cudaEventRecord(ex->ev_group[ex->n_pending], compute->s));
  pd.slab_first = slab_first; pd.slab_count = slab_count; pd.stride = stride; pd.seq = ++ex->seq;
  if (ex->trace && ex->n_marks + ex->n_pending < 16) VRHI_CUDA(cudaEventRecord(ex->t_computed[ex->n_marks + ex->n_pending], compute->s));
  ++ex->n_pending;
  return VRHI_OK;
}

int vrhi_exchange_complete(vrhi_exchange ex, vrhi_stream stream) {
  if (!ex || !stream) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (stream->dev != ex->grp->dev) return fail(VRHI_ERR_INVALID, "the stream belongs to another device than the group");
  stream->escape_chain = 0;
  ex->steps++;
  if (ex->grp->world == 1) return VRHI_OK;
  VRHI_TRY(set_dev(ex->grp->dev));
  VRHI_TRY(flush_pending(ex));
  VRHI_CUDA(cudaEventRecord(ex->ev_arrive, ex->arrive->s));
  VRHI_CUDA(cudaStreamWaitEvent(stream->s, ex->ev_arrive, 0));
  for (uint32_t k = 0; k < ex->n_push; ++k) {
    VRHI_CUDA(cudaEventRecord(ex->ev_push[k], ex->push[k]->s));
    VRHI_CUDA(cudaStreamWaitEvent(stream->s, ex->ev_push[k], 0));
  }
  ex->cur ^= 1u;
  if (ex->trace) {
    VRHI_CUDA(cudaEventRecord(ex->t_done, stream->s));
    ex->last_marks = ex->n_marks;
    ex->n_marks = 0;
  }
  return VRHI_OK;
}

int vrhi_exchange_check(vrhi_exchange ex) {
  if (!ex) return fail(VRHI_ERR_INVALID, "NULL exchange");
  if (ex->grp->world == 1) return VRHI_OK;
  VRHI_TRY(set_dev(ex->grp->dev));
  VRHI_TRY(flush_pending(ex));
  for (uint32_t k = 0; k < ex->n_push; ++k) VRHI_TRY(vrhi_stream_synchronize(ex->push[k]));
  int rc = vrhi_stream_check(ex->arrive);
  if (ex->trace && ex->last_marks && cudaEventSynchronize(ex->t_done) == cudaSuccess) {
    // the last completed step, milliseconds after its first group was computed
    fprintf(stderr, "vrhi_exchange rank %u, last step:", ex->grp->rank);
    for (uint32_t k = 0; k < ex->last_marks; ++k) {
      float c = 0.f, p = 0.f, w = 0.f;
      cudaEventElapsedTime(&c, ex->t_computed[0], ex->t_computed[k]);
      cudaEventElapsedTime(&p, ex->t_computed[0], ex->t_pushed[k]);
      cudaEventElapsedTime(&w, ex->t_computed[0], ex->t_widened[k]);
      fprintf(stderr, " [group %u computed %.3f sent %.3f widened %.3f]", k, c, p, w);
    }
    float d = 0.f;
    cudaEventElapsedTime(&d, ex->t_computed[0], ex->t_done);
    fprintf(stderr, " complete %.3f\n", d);
  }
  return rc;
}

int vrhi_exchange_launch_count(vrhi_exchange ex, uint64_t *out_count) {
  if (!ex || !out_count) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_count = 0;
  if (ex->grp->world > 1) {
    *out_count = ex->arrive->launches;
    for (uint32_t k = 0; k < ex->n_push; ++k) *out_count += ex->push[k]->launches;
  }
  return VRHI_OK;
}

}  // extern "C"
