// Device, buffer, stream, event, error and operator-registry half of libvrhi.so.
// Stands in for the runtime services fractal.py gets from Taichi (fractal.py:5 ti.init,
// :8 ti.field, :16 kernel registration, :31 launch); see include/vrhi.h.
#include <cstring>
#include <new>

#include "vrhi_internal.h"

namespace vrhi {

static thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

void clear_error() { g_last_error.clear(); }

static int set_device(vrhi_device_t *dev) {
  VRHI_CUDA(cudaSetDevice(dev->ordinal));
  return VRHI_OK;
}

int stream_arena(vrhi_stream_t *st, size_t payload, uint32_t **ctrl, char **payload_ptr) {
  if (!st->arena || st->arena_payload < payload) {
    VRHI_TRY(set_device(st->dev));
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    VRHI_CUDA(cudaStreamIsCapturing(st->s, &cap));
    if (cap != cudaStreamCaptureStatusNone)
      return fail(VRHI_ERR_INVALID, "this launch needs %zu bytes of stream scratch that do not exist yet; run the operator once on the stream before recording it", payload);
    // at least twice the old size, so that a stream outgrows its arena a bounded number of times
    size_t want = payload < (size_t(4) << 20) ? (size_t(4) << 20) : payload;
    if (st->arena && want < 2 * st->arena_payload) want = 2 * st->arena_payload;
    if (st->arena && st->n_retired >= (int)(sizeof st->retired / sizeof st->retired[0]))
      return fail(VRHI_ERR_OOM, "the stream's scratch has been regrown too often");
    void *p = nullptr;
    VRHI_CUDA(cudaMalloc(&p, kCtrlBytes + want));
    if (st->arena) {
      // The control block moves with the stream: a status a kernel has recorded (or is about to, the copy
      // is ordered behind it) is not lost.  The old arena is retired, not freed: recorded sequences still point into it.
      VRHI_CUDA(cudaMemcpyAsync(p, st->arena, kCtrlBytes, cudaMemcpyDeviceToDevice, st->s));
      VRHI_CUDA(cudaMemsetAsync(st->arena, 0, sizeof(uint32_t), st->s));  // the status word went along: report it once
      st->retired[st->n_retired++] = st->arena;
      st->escape_chain = 0;  // the ring of work counters moved: the next escape-time launch starts a new run
    } else {
      VRHI_CUDA(cudaMemsetAsync(p, 0, kCtrlBytes, st->s));
    }
    st->arena = static_cast<char *>(p);
    st->arena_payload = want;
  }
  if (ctrl) *ctrl = reinterpret_cast<uint32_t *>(st->arena);
  if (payload_ptr) *payload_ptr = st->arena + kCtrlBytes;
  return VRHI_OK;
}

static const OpDef kOps[] = {
    {"escape_time", "args: image(OUTPUT|IMAGE u32/u16/f32 [height][width])[, wire(OUTPUT|IMAGE u16 [height][width])[, bytes(OUTPUT|IMAGE u8 [height][width])]]; params: vrhi_escape_params",
     launch_escape_time},
    {"fused_map", "args: a,x,y(INPUT f32[n]), out(OUTPUT f32[n]); params: vrhi_map_params", launch_fused_map},
    {"map_tape", "args: inputs..., outputs...; params: vrhi_tape_params", launch_map_tape},
    {"row_sum", "args: in(INPUT f32[rows][cols]), out(OUTPUT f32[rows]); params: vrhi_rows_params", launch_row_sum},
    {"row_max", "args: in(INPUT f32[rows][cols]), out(OUTPUT f32[rows]); params: vrhi_rows_params", launch_row_max},
    {"row_softmax", "args: in(INPUT f32[rows][cols]), out(OUTPUT f32[rows][cols]); params: vrhi_rows_params",
     launch_row_softmax},
    {"row_stats_softmax",
     "args: in(INPUT), sum(OUTPUT f32[rows]), max(OUTPUT f32[rows]), softmax(OUTPUT f32[rows][cols]); params: "
     "vrhi_rows_params",
     launch_row_stats_softmax},
    {"col_sum", "args: in(INPUT f32[rows][cols]), out(OUTPUT f32[cols]); params: vrhi_rows_params", launch_col_sum},
    {"mse_tanh_fwd", "args: W,x,b,t(INPUT), loss(OUTPUT f32[1]); params: vrhi_mse_params", launch_mse_tanh_fwd},
    {"mse_tanh_bwd", "args: W,x,b,t(INPUT), dW,dx,db(OUTPUT)[, loss(OUTPUT f32[1])]; params: vrhi_mse_params",
     launch_mse_tanh_bwd},
    {"fp32_probe", "args: out(OUTPUT >=4 bytes); params: vrhi_probe_params", launch_fp32_probe},
    {"vertex_transform",
     "args: pos(INPUT f32[n][3]), model,view,proj(UNIFORM f32[16] row-major), gl_position(OUTPUT f32[n][4]), "
     "varying(VARYING f32[n][3]); params: vrhi_map_params",
     launch_vertex_transform},
    {"flat_color", "args: color(UNIFORM f32[3]), fragments(IMAGE f32[n][4]); params: vrhi_map_params", launch_flat_color},
    {"widen_rows_u16", "args: wire(u16 [height][width]), image(OUTPUT|IMAGE u32 [height][width]); params: vrhi_widen_params",
     launch_widen_rows_u16},
    {"widen_rows_u8", "args: bytes(u8 [height][width]), image(OUTPUT|IMAGE u32 [height][width]), the ranks' wire images (u16 [height][width]) in rank order; params: vrhi_widen_params",
     launch_widen_rows_u8},
    {"gather_signal", "args: the peers' flag arrays (u32[world]); params: vrhi_gather_params", launch_gather_signal},
    {"gather_pull_u16", "args: flags(u32[world]), image(u32 [height][width]), the peers' wire images (u16 [height][width]) in rank order; params: vrhi_gather_params",
     launch_gather_pull_u16},
};
static const int kNumOps = int(sizeof(kOps) / sizeof(kOps[0]));

static const char *const kSemantic[] = {"input",  "output", "uniform", "uniform_constant",
                                        "storage_buffer", "image", "varying"};

}  // namespace vrhi

using namespace vrhi;

extern "C" {

const char *vrhi_last_error(void) { return g_last_error.c_str(); }
int vrhi_version(void) { return VRHI_VERSION; }

int vrhi_arg_class_from_semantic(const char *semantic, int *out_class) {
  if (!semantic || !out_class) return fail(VRHI_ERR_INVALID, "NULL argument");
  for (int k = 0; k <= VRHI_VARYING; ++k)
    if (strcmp(semantic, kSemantic[k]) == 0) {
      *out_class = k;
      return VRHI_OK;
    }
  return fail(VRHI_ERR_NOT_FOUND, "unknown vernon.semantic '%s'", semantic);
}

const char *vrhi_arg_class_name(int arg_class) {
  return (arg_class >= 0 && arg_class <= VRHI_VARYING) ? kSemantic[arg_class] : nullptr;
}

/* ---------------------------------------------------------------- device ---------------- */

int vrhi_device_count(int *out_count) {
  if (!out_count) return fail(VRHI_ERR_INVALID, "NULL out_count");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    *out_count = 0;
    return fail(VRHI_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e));
  }
  *out_count = n;
  return VRHI_OK;
}

int vrhi_device_create(int ordinal, vrhi_device *out_dev) {
  if (!out_dev) return fail(VRHI_ERR_INVALID, "NULL out_dev");
  *out_dev = nullptr;
  int n = 0;
  VRHI_TRY(vrhi_device_count(&n));
  if (ordinal < 0 || ordinal >= n) return fail(VRHI_ERR_INVALID, "device ordinal %d out of range [0,%d)", ordinal, n);
  vrhi_device_t *d = new (std::nothrow) vrhi_device_t();
  if (!d) return fail(VRHI_ERR_OOM, "host allocation failed");
  d->ordinal = ordinal;
  cudaError_t e = cudaSetDevice(ordinal);
  if (e == cudaSuccess) e = cudaGetDeviceProperties(&d->prop, ordinal);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d->sm_clock_khz, cudaDevAttrClockRate, ordinal);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d->mem_clock_khz, cudaDevAttrMemoryClockRate, ordinal);
  if (e != cudaSuccess) {
    delete d;
    return fail(VRHI_ERR_CUDA, "opening device %d failed: %s", ordinal, cudaGetErrorString(e));
  }
  if (d->prop.major < 10) {
    int maj = d->prop.major, min = d->prop.minor;
    delete d;
    return fail(VRHI_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library carries sm_100a code only", ordinal, maj, min);
  }
  vrhi_stream_t *s = new (std::nothrow) vrhi_stream_t();
  if (!s) {
    delete d;
    return fail(VRHI_ERR_OOM, "host allocation failed");
  }
  s->dev = d;
  s->s = nullptr;  // legacy default stream
  s->owned = false;
  d->default_stream = s;
  *out_dev = d;
  return VRHI_OK;
}

int vrhi_device_destroy(vrhi_device dev) {
  if (!dev) return VRHI_OK;
  if (dev->default_stream) {
    if (dev->default_stream->arena) {
      cudaSetDevice(dev->ordinal);
      cudaFree(dev->default_stream->arena);
      for (int k = 0; k < dev->default_stream->n_retired; ++k) cudaFree(dev->default_stream->retired[k]);
    }
    delete dev->default_stream;
  }
  delete dev;
  return VRHI_OK;
}

int vrhi_device_props_get(vrhi_device dev, vrhi_device_props *out) {
  if (!dev || !out) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (out->size < sizeof(uint32_t) * 2) return fail(VRHI_ERR_SIZE, "vrhi_device_props.size not set");
  vrhi_device_props p{};
  p.size = sizeof p;
  p.ordinal = dev->ordinal;
  p.sm_count = dev->prop.multiProcessorCount;
  p.cc_major = dev->prop.major;
  p.cc_minor = dev->prop.minor;
  p.sm_clock_khz = dev->sm_clock_khz;
  p.mem_clock_khz = dev->mem_clock_khz;
  p.l2_bytes = dev->prop.l2CacheSize;
  p.smem_per_block_optin = (int32_t)dev->prop.sharedMemPerBlockOptin;
  p.total_mem_bytes = dev->prop.totalGlobalMem;
  strncpy(p.name, dev->prop.name, sizeof p.name - 1);
  size_t n = out->size < sizeof p ? out->size : sizeof p;
  uint32_t declared = out->size;
  memcpy(out, &p, n);
  out->size = declared < sizeof p ? declared : (uint32_t)sizeof p;
  return VRHI_OK;
}

int vrhi_device_synchronize(vrhi_device dev) {
  if (!dev) return fail(VRHI_ERR_INVALID, "NULL device");
  VRHI_TRY(set_device(dev));
  VRHI_CUDA(cudaDeviceSynchronize());
  return VRHI_OK;
}

int vrhi_device_set_alloc_limit(vrhi_device dev, uint64_t bytes) {
  if (!dev) return fail(VRHI_ERR_INVALID, "NULL device");
  dev->limit = bytes;
  return VRHI_OK;
}

int vrhi_device_allocated(vrhi_device dev, uint64_t *out_bytes) {
  if (!dev || !out_bytes) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_bytes = dev->allocated;
  return VRHI_OK;
}

/* ---------------------------------------------------------------- buffers --------------- */

static int check_class(int cls) {
  if (cls < VRHI_INPUT || cls > VRHI_VARYING) return fail(VRHI_ERR_INVALID, "argument class %d out of range", cls);
  return VRHI_OK;
}

int vrhi_buffer_create(vrhi_device dev, uint64_t bytes, int arg_class, vrhi_buffer *out_buf) {
  if (!dev || !out_buf) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_buf = nullptr;
  VRHI_TRY(check_class(arg_class));
  if (bytes == 0) return fail(VRHI_ERR_SIZE, "zero-sized buffer");
  if (dev->limit && dev->allocated + bytes > dev->limit)
    return fail(VRHI_ERR_OOM, "allocation of %llu bytes exceeds the device handle's limit (%llu held, limit %llu)",
                (unsigned long long)bytes, (unsigned long long)dev->allocated, (unsigned long long)dev->limit);
  VRHI_TRY(set_device(dev));
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(e == cudaErrorMemoryAllocation ? VRHI_ERR_OOM : VRHI_ERR_CUDA, "cudaMalloc(%llu) failed: %s",
                (unsigned long long)bytes, cudaGetErrorString(e));
  }
  vrhi_buffer_t *b = new (std::nothrow) vrhi_buffer_t{dev, p, bytes, arg_class, true};
  if (!b) {
    cudaFree(p);
    return fail(VRHI_ERR_OOM, "host allocation failed");
  }
  dev->allocated += bytes;
  *out_buf = b;
  return VRHI_OK;
}

int vrhi_buffer_wrap(vrhi_device dev, void *device_ptr, uint64_t bytes, int arg_class, vrhi_buffer *out_buf) {
  if (!dev || !out_buf || !device_ptr) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_buf = nullptr;
  VRHI_TRY(check_class(arg_class));
  if (bytes == 0) return fail(VRHI_ERR_SIZE, "zero-sized buffer");
  if (reinterpret_cast<uintptr_t>(device_ptr) % 16) return fail(VRHI_ERR_SIZE, "wrapped pointer is not 16-byte aligned");
  vrhi_buffer_t *b = new (std::nothrow) vrhi_buffer_t{dev, device_ptr, bytes, arg_class, false};
  if (!b) return fail(VRHI_ERR_OOM, "host allocation failed");
  *out_buf = b;
  return VRHI_OK;
}

int vrhi_buffer_destroy(vrhi_buffer buf) {
  if (!buf) return VRHI_OK;
  int rc = VRHI_OK;
  if (buf->ipc) {
    cudaSetDevice(buf->dev->ordinal);
    cudaError_t e = cudaIpcCloseMemHandle(buf->ptr);
    if (e != cudaSuccess) rc = fail(VRHI_ERR_CUDA, "cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
  } else if (buf->owned) {
    cudaSetDevice(buf->dev->ordinal);
    cudaError_t e = cudaFree(buf->ptr);
    if (e != cudaSuccess) rc = fail(VRHI_ERR_CUDA, "cudaFree failed: %s", cudaGetErrorString(e));
    buf->dev->allocated -= buf->bytes;
  }
  delete buf;
  return rc;
}

int vrhi_buffer_size(vrhi_buffer buf, uint64_t *out_bytes) {
  if (!buf || !out_bytes) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_bytes = buf->bytes;
  return VRHI_OK;
}

int vrhi_buffer_class(vrhi_buffer buf, int *out_class) {
  if (!buf || !out_class) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_class = buf->cls;
  return VRHI_OK;
}

int vrhi_buffer_device_ptr(vrhi_buffer buf, void **out_ptr) {
  if (!buf || !out_ptr) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_ptr = buf->ptr;
  return VRHI_OK;
}

static int range_ok(vrhi_buffer buf, uint64_t offset, uint64_t bytes) {
  if (offset > buf->bytes || bytes > buf->bytes - offset)
    return fail(VRHI_ERR_SIZE, "range [%llu, +%llu) exceeds the buffer (%llu bytes)", (unsigned long long)offset,
                (unsigned long long)bytes, (unsigned long long)buf->bytes);
  return VRHI_OK;
}

static int copy(vrhi_buffer buf, uint64_t offset, void *host, uint64_t bytes, vrhi_stream stream, bool up) {
  if (!buf || (!host && bytes)) return fail(VRHI_ERR_INVALID, "NULL argument");
  VRHI_TRY(range_ok(buf, offset, bytes));
  if (stream && stream->dev != buf->dev) return fail(VRHI_ERR_INVALID, "stream and buffer belong to different devices");
  if (bytes == 0) return VRHI_OK;
  VRHI_TRY(set_device(buf->dev));
  char *d = static_cast<char *>(buf->ptr) + offset;
  if (stream) {
    stream->escape_chain = 0;
    VRHI_CUDA(cudaMemcpyAsync(up ? (void *)d : host, up ? (const void *)host : (const void *)d, bytes,
                              up ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, stream->s));
  } else {
    VRHI_CUDA(cudaMemcpy(up ? (void *)d : host, up ? (const void *)host : (const void *)d, bytes,
                         up ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost));
  }
  return VRHI_OK;
}

int vrhi_buffer_upload(vrhi_buffer buf, uint64_t offset, const void *host, uint64_t bytes, vrhi_stream stream) {
  if (buf && (buf->cls == VRHI_OUTPUT)) { /* uploading into an OUTPUT buffer is allowed (initial value) */ }
  return copy(buf, offset, const_cast<void *>(host), bytes, stream, true);
}

int vrhi_buffer_download(vrhi_buffer buf, uint64_t offset, void *host, uint64_t bytes, vrhi_stream stream) {
  return copy(buf, offset, host, bytes, stream, false);
}

int vrhi_buffer_fill_u8(vrhi_buffer buf, uint64_t offset, int value, uint64_t bytes, vrhi_stream stream) {
  if (!buf) return fail(VRHI_ERR_INVALID, "NULL buffer");
  VRHI_TRY(range_ok(buf, offset, bytes));
  if (bytes == 0) return VRHI_OK;
  VRHI_TRY(set_device(buf->dev));
  char *d = static_cast<char *>(buf->ptr) + offset;
  if (stream) stream->escape_chain = 0;
  if (stream)
    VRHI_CUDA(cudaMemsetAsync(d, value, bytes, stream->s));
  else
    VRHI_CUDA(cudaMemset(d, value, bytes));
  return VRHI_OK;
}

int vrhi_host_alloc(uint64_t bytes, void **out_host) {
  if (!out_host) return fail(VRHI_ERR_INVALID, "NULL out_host");
  *out_host = nullptr;
  if (bytes == 0) return fail(VRHI_ERR_SIZE, "zero-sized allocation");
  cudaError_t e = cudaMallocHost(out_host, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(VRHI_ERR_OOM, "cudaMallocHost(%llu) failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
  }
  return VRHI_OK;
}

int vrhi_host_free(void *host) {
  if (!host) return VRHI_OK;
  VRHI_CUDA(cudaFreeHost(host));
  return VRHI_OK;
}

int vrhi_buffer_copy_2d(vrhi_buffer dst, uint64_t dst_offset, uint64_t dst_pitch, vrhi_buffer src, uint64_t src_offset,
                        uint64_t src_pitch, uint64_t width_bytes, uint64_t rows, vrhi_stream stream) {
  if (!dst || !src) return fail(VRHI_ERR_INVALID, "NULL buffer");
  if (width_bytes == 0 || rows == 0) return VRHI_OK;
  if (rows > 1 && (dst_pitch < width_bytes || src_pitch < width_bytes)) return fail(VRHI_ERR_SIZE, "pitch smaller than the row width");
  const uint64_t dst_span = (rows - 1) * dst_pitch + width_bytes, src_span = (rows - 1) * src_pitch + width_bytes;
  if (dst_offset > dst->bytes || dst_span > dst->bytes - dst_offset) return fail(VRHI_ERR_SIZE, "copy exceeds the destination buffer");
  if (src_offset > src->bytes || src_span > src->bytes - src_offset) return fail(VRHI_ERR_SIZE, "copy exceeds the source buffer");
  if (dst->cls == VRHI_INPUT || dst->cls == VRHI_UNIFORM || dst->cls == VRHI_UNIFORM_CONSTANT)
    return fail(VRHI_ERR_INVALID, "copy destination is read-only (class %s)", vrhi_arg_class_name(dst->cls));
  VRHI_TRY(set_device(src->dev));
  cudaStream_t s = stream ? stream->s : nullptr;
  if (stream) stream->escape_chain = 0;
  char *d = static_cast<char *>(dst->ptr) + dst_offset;
  const char *sp = static_cast<const char *>(src->ptr) + src_offset;
  if (rows == 1)
    VRHI_CUDA(cudaMemcpyAsync(d, sp, width_bytes, cudaMemcpyDeviceToDevice, s));
  else
    VRHI_CUDA(cudaMemcpy2DAsync(d, dst_pitch, sp, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice, s));
  return VRHI_OK;
}

int vrhi_buffer_ipc_export(vrhi_buffer buf, void *out_handle) {
  if (!buf || !out_handle) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!buf->owned) return fail(VRHI_ERR_INVALID, "only buffers this library allocated can be exported");
  static_assert(sizeof(cudaIpcMemHandle_t) == VRHI_IPC_HANDLE_BYTES, "handle size");
  VRHI_TRY(set_device(buf->dev));
  cudaIpcMemHandle_t h;
  VRHI_CUDA(cudaIpcGetMemHandle(&h, buf->ptr));
  memcpy(out_handle, &h, sizeof h);
  return VRHI_OK;
}

int vrhi_buffer_ipc_open(vrhi_device dev, const void *handle, uint64_t bytes, int arg_class, vrhi_buffer *out_buf) {
  if (!dev || !handle || !out_buf) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_buf = nullptr;
  VRHI_TRY(check_class(arg_class));
  if (bytes == 0) return fail(VRHI_ERR_SIZE, "zero-sized buffer");
  VRHI_TRY(set_device(dev));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void *p = nullptr;
  VRHI_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  vrhi_buffer_t *b = new (std::nothrow) vrhi_buffer_t{dev, p, bytes, arg_class, false, true};
  if (!b) {
    cudaIpcCloseMemHandle(p);
    return fail(VRHI_ERR_OOM, "host allocation failed");
  }
  *out_buf = b;
  return VRHI_OK;
}

/* ---------------------------------------------------------------- streams / events ------ */

int vrhi_stream_create(vrhi_device dev, vrhi_stream *out_stream) {
  if (!dev || !out_stream) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_stream = nullptr;
  VRHI_TRY(set_device(dev));
  cudaStream_t s;
  VRHI_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  vrhi_stream_t *st = new (std::nothrow) vrhi_stream_t{dev, s, true, nullptr, 0, 0};
  if (!st) {
    cudaStreamDestroy(s);
    return fail(VRHI_ERR_OOM, "host allocation failed");
  }
  *out_stream = st;
  return VRHI_OK;
}

int vrhi_stream_wrap(vrhi_device dev, void *cuda_stream, vrhi_stream *out_stream) {
  if (!dev || !out_stream) return fail(VRHI_ERR_INVALID, "NULL argument");
  vrhi_stream_t *st = new (std::nothrow) vrhi_stream_t{dev, static_cast<cudaStream_t>(cuda_stream), false, nullptr, 0, 0};
  if (!st) return fail(VRHI_ERR_OOM, "host allocation failed");
  *out_stream = st;
  return VRHI_OK;
}

int vrhi_stream_destroy(vrhi_stream stream) {
  if (!stream) return VRHI_OK;
  if (stream == stream->dev->default_stream) return fail(VRHI_ERR_INVALID, "the device's default stream is not destroyed by the caller");
  cudaSetDevice(stream->dev->ordinal);
  int rc = VRHI_OK;
  if (stream->arena) {
    cudaStreamSynchronize(stream->s);
    cudaFree(stream->arena);
    for (int k = 0; k < stream->n_retired; ++k) cudaFree(stream->retired[k]);
  }
  if (stream->fork_event) cudaEventDestroy(stream->fork_event);
  if (stream->owned) {
    cudaError_t e = cudaStreamDestroy(stream->s);
    if (e != cudaSuccess) rc = fail(VRHI_ERR_CUDA, "cudaStreamDestroy failed: %s", cudaGetErrorString(e));
  }
  delete stream;
  return rc;
}

int vrhi_stream_synchronize(vrhi_stream stream) {
  if (!stream) return fail(VRHI_ERR_INVALID, "NULL stream");
  VRHI_TRY(set_device(stream->dev));
  VRHI_CUDA(cudaStreamSynchronize(stream->s));
  return VRHI_OK;
}

int vrhi_stream_check(vrhi_stream stream) {
  if (!stream) return fail(VRHI_ERR_INVALID, "NULL stream");
  VRHI_TRY(vrhi_stream_synchronize(stream));
  if (!stream->arena) return VRHI_OK;
  // the current arena, then the retired ones: kernels of a sequence recorded before the scratch grew report there
  for (int k = -1; k < stream->n_retired; ++k) {
    char *arena = k < 0 ? stream->arena : stream->retired[k];
    int32_t status = 0;
    VRHI_CUDA(cudaMemcpy(&status, arena, sizeof status, cudaMemcpyDeviceToHost));
    if (status != 0) {
      VRHI_CUDA(cudaMemset(arena, 0, sizeof status));
      return fail(status, "a kernel on this stream recorded device status %d", status);
    }
  }
  return VRHI_OK;
}

int vrhi_stream_launch_count(vrhi_stream stream, uint64_t *out_count) {
  if (!stream || !out_count) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_count = stream->launches;
  return VRHI_OK;
}

int vrhi_event_create(vrhi_device dev, vrhi_event *out_event) {
  if (!dev || !out_event) return fail(VRHI_ERR_INVALID, "NULL argument");
  *out_event = nullptr;
  VRHI_TRY(set_device(dev));
  cudaEvent_t e;
  VRHI_CUDA(cudaEventCreate(&e));
  vrhi_event_t *ev = new (std::nothrow) vrhi_event_t{dev, e};
  if (!ev) {
    cudaEventDestroy(e);
    return fail(VRHI_ERR_OOM, "host allocation failed");
  }
  *out_event = ev;
  return VRHI_OK;
}

int vrhi_event_destroy(vrhi_event event) {
  if (!event) return VRHI_OK;
  cudaSetDevice(event->dev->ordinal);
  cudaEventDestroy(event->e);
  delete event;
  return VRHI_OK;
}

int vrhi_event_record(vrhi_event event, vrhi_stream stream) {
  if (!event) return fail(VRHI_ERR_INVALID, "NULL event");
  VRHI_TRY(set_device(event->dev));
  if (stream) stream->escape_chain = 0;
  VRHI_CUDA(cudaEventRecord(event->e, stream ? stream->s : nullptr));
  return VRHI_OK;
}

int vrhi_event_synchronize(vrhi_event event) {
  if (!event) return fail(VRHI_ERR_INVALID, "NULL event");
  VRHI_CUDA(cudaEventSynchronize(event->e));
  return VRHI_OK;
}

int vrhi_event_elapsed_ms(vrhi_event start, vrhi_event stop, float *out_ms) {
  if (!start || !stop || !out_ms) return fail(VRHI_ERR_INVALID, "NULL argument");
  VRHI_CUDA(cudaEventElapsedTime(out_ms, start->e, stop->e));
  return VRHI_OK;
}

int vrhi_tape_jit_stats(uint64_t *out_compiled, uint64_t *out_launches, int *out_compiler_version, int *out_built_version) {
  tape_jit_counters(out_compiled, out_launches, out_compiler_version, out_built_version);
  return VRHI_OK;
}

int vrhi_tape_source(const vrhi_tape_params *params, char *buffer, uint64_t capacity, uint64_t *out_needed) {
  if (!params) return fail(VRHI_ERR_INVALID, "NULL argument");
  vrhi_tape_params q;
  VRHI_TRY(read_params(params, params->size, &q));
  if (q.n_inputs > VRHI_TAPE_MAX_INPUTS || q.n_outputs == 0 || q.n_outputs > VRHI_TAPE_MAX_OUTPUTS || q.n_instr > VRHI_TAPE_MAX_INSTR)
    return fail(VRHI_ERR_INVALID, "tape outside the limits");
  for (uint32_t t = 0; t < q.n_instr; ++t)
    if (q.instr[t].op >= VRHI_T_OPCOUNT) return fail(VRHI_ERR_INVALID, "instruction %u has unknown opcode %u", t, q.instr[t].op);
  const std::string src = tape_jit_source(q);
  if (out_needed) *out_needed = src.size() + 1;
  if (buffer && capacity) {
    const size_t n = src.size() < capacity - 1 ? src.size() : (size_t)capacity - 1;
    memcpy(buffer, src.data(), n);
    buffer[n] = 0;
  }
  return VRHI_OK;
}

/* ---------------------------------------------------------------- recorded sequences ---- */

int vrhi_sequence_begin(vrhi_stream stream) {
  if (!stream) return fail(VRHI_ERR_INVALID, "NULL stream");
  if (stream->recording) return fail(VRHI_ERR_INVALID, "the stream is already recording");
  VRHI_TRY(set_device(stream->dev));
  // thread-local mode: an allocation or synchronisation attempted by THIS thread while recording
  // fails loudly instead of corrupting the recording; other threads are unaffected
  VRHI_CUDA(cudaStreamBeginCapture(stream->s, cudaStreamCaptureModeThreadLocal));
  stream->recording = true;
  stream->record_mark = stream->launches;
  stream->escape_chain = 0;  // a recording may be replayed behind anything: its first launch is ordered
  return VRHI_OK;
}

int vrhi_sequence_fork(vrhi_stream stream, vrhi_stream side) {
  if (!stream || !side) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!stream->recording || stream->record_main) return fail(VRHI_ERR_INVALID, "fork needs the stream on which the recording began");
  if (side == stream || side->dev != stream->dev) return fail(VRHI_ERR_INVALID, "the side stream must be another stream of the same device");
  if (side->recording) return fail(VRHI_ERR_INVALID, "the side stream is already recording");
  if (stream->n_record_sides >= 4) return fail(VRHI_ERR_UNSUPPORTED, "at most 4 side streams per recording");
  VRHI_TRY(set_device(stream->dev));
  if (!stream->fork_event) VRHI_CUDA(cudaEventCreateWithFlags(&stream->fork_event, cudaEventDisableTiming));
  VRHI_CUDA(cudaEventRecord(stream->fork_event, stream->s));
  VRHI_CUDA(cudaStreamWaitEvent(side->s, stream->fork_event, 0));  // the side stream joins the capture here
  side->recording = true;
  side->escape_chain = 0;
  stream->escape_chain = 0;
  side->record_main = stream;
  side->record_mark = side->launches;
  stream->record_sides[stream->n_record_sides++] = side;
  return VRHI_OK;
}

int vrhi_sequence_end(vrhi_stream stream, vrhi_sequence *inout_seq) {
  if (!stream || !inout_seq) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!stream->recording) return fail(VRHI_ERR_INVALID, "the stream is not recording");
  if (stream->record_main) return fail(VRHI_ERR_INVALID, "end the recording on the stream it began on");
  VRHI_TRY(set_device(stream->dev));
  stream->recording = false;
  stream->escape_chain = 0;  // nothing of the recording precedes the next launch on the stream
  uint64_t kernels = stream->launches - stream->record_mark;
  stream->launches = stream->record_mark;  // nothing ran
  for (int k = 0; k < stream->n_record_sides; ++k) {
    vrhi_stream_t *side = stream->record_sides[k];
    // rejoin: the recording ends only after everything recorded on the side stream
    if (!side->fork_event) cudaEventCreateWithFlags(&side->fork_event, cudaEventDisableTiming);
    if (side->fork_event) {
      cudaEventRecord(side->fork_event, side->s);
      cudaStreamWaitEvent(stream->s, side->fork_event, 0);
    }
    kernels += side->launches - side->record_mark;
    side->launches = side->record_mark;
    side->recording = false;
    side->escape_chain = 0;
    side->record_main = nullptr;
  }
  stream->n_record_sides = 0;
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(stream->s, &g);
  if (e != cudaSuccess || !g) {
    if (g) cudaGraphDestroy(g);
    return fail(VRHI_ERR_CUDA, "the recording was invalidated: %s", cudaGetErrorString(e));
  }
  vrhi_sequence_t *seq = *inout_seq;
  if (seq) {
    cudaGraphExecUpdateResultInfo info{};
    e = cudaGraphExecUpdate(seq->exec, g, &info);
    if (e == cudaSuccess) {
      seq->kernels = kernels;
      seq->retargets++;
      cudaGraphDestroy(g);
      return VRHI_OK;
    }
    (void)cudaGetLastError();  // a different shape of recording: rebuild below
    cudaGraphExecDestroy(seq->exec);
    seq->exec = nullptr;
    seq->rebuilds++;
  } else {
    seq = new (std::nothrow) vrhi_sequence_t{stream->dev, nullptr, 0, 0, 0};
    if (!seq) {
      cudaGraphDestroy(g);
      return fail(VRHI_ERR_OOM, "host allocation failed");
    }
  }
  e = cudaGraphInstantiate(&seq->exec, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) {
    if (!*inout_seq) delete seq; else seq->exec = nullptr;
    return fail(VRHI_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  }
  seq->kernels = kernels;
  *inout_seq = seq;
  return VRHI_OK;
}

int vrhi_sequence_launch(vrhi_sequence seq, vrhi_stream stream) {
  if (!seq || !stream) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (!seq->exec) return fail(VRHI_ERR_INVALID, "the sequence holds no recording");
  if (seq->dev != stream->dev) return fail(VRHI_ERR_INVALID, "the sequence was recorded on another device");
  VRHI_TRY(set_device(stream->dev));
  VRHI_CUDA(cudaGraphLaunch(seq->exec, stream->s));
  stream->escape_chain = 0;
  stream->launches += seq->kernels;
  return VRHI_OK;
}

int vrhi_sequence_stats(vrhi_sequence seq, uint64_t *out_kernels, uint64_t *out_retargets, uint64_t *out_rebuilds) {
  if (!seq) return fail(VRHI_ERR_INVALID, "NULL sequence");
  if (out_kernels) *out_kernels = seq->kernels;
  if (out_retargets) *out_retargets = seq->retargets;
  if (out_rebuilds) *out_rebuilds = seq->rebuilds;
  return VRHI_OK;
}

int vrhi_sequence_destroy(vrhi_sequence seq) {
  if (!seq) return VRHI_OK;
  cudaSetDevice(seq->dev->ordinal);
  if (seq->exec) cudaGraphExecDestroy(seq->exec);
  delete seq;
  return VRHI_OK;
}

int vrhi_stream_wait_event(vrhi_stream stream, vrhi_event event) {
  if (!stream || !event) return fail(VRHI_ERR_INVALID, "NULL argument");
  VRHI_TRY(set_device(stream->dev));
  stream->escape_chain = 0;
  VRHI_CUDA(cudaStreamWaitEvent(stream->s, event->e, 0));
  return VRHI_OK;
}

/* ---------------------------------------------------------------- operators ------------- */

int vrhi_op_count(int *out_count) {
  if (!out_count) return fail(VRHI_ERR_INVALID, "NULL out_count");
  *out_count = kNumOps;
  return VRHI_OK;
}

int vrhi_op_name(int op, const char **out_name) {
  if (!out_name) return fail(VRHI_ERR_INVALID, "NULL out_name");
  if (op < 0 || op >= kNumOps) return fail(VRHI_ERR_NOT_FOUND, "operator id %d out of range", op);
  *out_name = kOps[op].name;
  return VRHI_OK;
}

int vrhi_op_signature(int op, const char **out_text) {
  if (!out_text) return fail(VRHI_ERR_INVALID, "NULL out_text");
  if (op < 0 || op >= kNumOps) return fail(VRHI_ERR_NOT_FOUND, "operator id %d out of range", op);
  *out_text = kOps[op].signature;
  return VRHI_OK;
}

int vrhi_op_lookup(const char *name, int *out_op) {
  if (!name || !out_op) return fail(VRHI_ERR_INVALID, "NULL argument");
  for (int k = 0; k < kNumOps; ++k)
    if (strcmp(kOps[k].name, name) == 0) {
      *out_op = k;
      return VRHI_OK;
    }
  return fail(VRHI_ERR_NOT_FOUND, "no operator named '%s'", name);
}

int vrhi_op_launch(vrhi_stream stream, int op, const vrhi_arg *args, int n_args, const void *params,
                   size_t params_size) {
  if (!stream) return fail(VRHI_ERR_INVALID, "NULL stream");
  if (op < 0 || op >= kNumOps) return fail(VRHI_ERR_NOT_FOUND, "operator id %d out of range", op);
  if (n_args < 0 || n_args > 16 || (n_args && !args)) return fail(VRHI_ERR_INVALID, "bad argument list");
  ArgView views[16];
  for (int k = 0; k < n_args; ++k) {
    const vrhi_arg &a = args[k];
    if (!a.buffer) return fail(VRHI_ERR_INVALID, "%s: argument %d has no buffer", kOps[op].name, k);
    if (a.buffer->dev != stream->dev) return fail(VRHI_ERR_INVALID, "%s: argument %d lives on another device", kOps[op].name, k);
    if (a.offset % 16) return fail(VRHI_ERR_SIZE, "%s: argument %d offset %llu is not a multiple of 16", kOps[op].name, k, (unsigned long long)a.offset);
    if (a.offset > a.buffer->bytes) return fail(VRHI_ERR_SIZE, "%s: argument %d offset beyond the buffer", kOps[op].name, k);
    uint64_t avail = a.buffer->bytes - a.offset;
    uint64_t bytes = a.bytes ? a.bytes : avail;
    if (bytes > avail) return fail(VRHI_ERR_SIZE, "%s: argument %d view exceeds the buffer", kOps[op].name, k);
    VRHI_TRY(check_class(a.arg_class));
    views[k] = ArgView{static_cast<char *>(a.buffer->ptr) + a.offset, bytes, a.arg_class, a.buffer->cls};
  }
  VRHI_TRY(set_device(stream->dev));
  return kOps[op].launch(stream, views, n_args, params, params_size);
}

/* ---------------------------------------------------------------- partitioning ---------- */

int vrhi_partition_rows(uint64_t total_rows, uint32_t chunk_rows, uint32_t world, uint32_t rank, int scheme,
                        vrhi_row_partition *out) {
  if (!out) return fail(VRHI_ERR_INVALID, "NULL out");
  if (world == 0 || rank >= world) return fail(VRHI_ERR_INVALID, "rank %u outside world %u", rank, world);
  if (total_rows == 0 || total_rows > 0xffffffffull) return fail(VRHI_ERR_SIZE, "row count out of range");
  vrhi_row_partition p{};
  if (scheme == VRHI_PART_CONTIGUOUS) {
    // one band per rank: band height = ceil(total/world) rounded up to chunk_rows (if given)
    uint64_t band = (total_rows + world - 1) / world;
    if (chunk_rows > 1) band = (band + chunk_rows - 1) / chunk_rows * chunk_rows;
    uint64_t begin = band * rank;
    p.chunk_rows = (uint32_t)band;
    p.chunk_first = rank;
    p.chunk_step = world;
    p.chunk_count = begin < total_rows ? 1u : 0u;
    p.rows_owned = begin < total_rows ? (total_rows - begin < band ? total_rows - begin : band) : 0;
  } else if (scheme == VRHI_PART_CYCLIC) {
    if (chunk_rows == 0) return fail(VRHI_ERR_INVALID, "cyclic partition needs chunk_rows > 0");
    uint64_t n_chunks = (total_rows + chunk_rows - 1) / chunk_rows;
    uint64_t mine = n_chunks > rank ? (n_chunks - rank + world - 1) / world : 0;
    p.chunk_rows = chunk_rows;
    p.chunk_first = rank;
    p.chunk_step = world;
    p.chunk_count = (uint32_t)mine;
    uint64_t rows = mine * chunk_rows;
    // the globally last chunk may be short; it belongs to rank (n_chunks-1) % world
    if (mine && (n_chunks - 1) % world == rank) rows -= n_chunks * chunk_rows - total_rows;
    p.rows_owned = rows;
  } else {
    return fail(VRHI_ERR_INVALID, "unknown partition scheme %d", scheme);
  }
  *out = p;
  return VRHI_OK;
}

int vrhi_partition_leading(uint64_t n, uint32_t world, uint32_t rank, uint64_t *out_begin, uint64_t *out_count) {
  if (!out_begin || !out_count) return fail(VRHI_ERR_INVALID, "NULL argument");
  if (world == 0 || rank >= world) return fail(VRHI_ERR_INVALID, "rank %u outside world %u", rank, world);
  uint64_t base = n / world, extra = n % world;
  *out_begin = base * rank + (rank < extra ? rank : extra);
  *out_count = base + (rank < extra ? 1 : 0);
  return VRHI_OK;
}

}  // extern "C"
