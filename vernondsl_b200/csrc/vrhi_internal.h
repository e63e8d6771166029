// Internal definitions shared by the translation units of libvrhi.so.  Not installed.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

struct vrhi_stream_t;

#include "vrhi.h"

struct vrhi_device_t {
  int ordinal;
  cudaDeviceProp prop;
  int sm_clock_khz, mem_clock_khz;
  uint64_t allocated, limit;
  vrhi_stream_t *default_stream;
};

struct vrhi_buffer_t {
  vrhi_device_t *dev;
  void *ptr;
  uint64_t bytes;
  int cls;
  bool owned;
  bool ipc;  // mapping of another process's allocation (closed, not freed, on destroy)
};

// Per-stream scratch arena.  Kernels launched on one stream are ordered, so they may share it.
// Layout: [0,256) control words (status, work counters), then `scratch_bytes` of payload.
struct vrhi_stream_t {
  vrhi_device_t *dev;
  cudaStream_t s;
  bool owned;
  char *arena;           // device memory, or nullptr until first use
  size_t arena_payload;  // payload bytes available behind the control block
  uint64_t launches;
  uint64_t record_mark;  // value of `launches` when recording began
  bool recording;
  vrhi_stream_t *record_main;  // side stream of a recording: the stream that owns it
  vrhi_stream_t *record_sides[4];
  int n_record_sides;
  cudaEvent_t fork_event;      // created on first use, reused
  // Arenas this stream has outgrown.  They stay allocated until the stream is destroyed: a recorded
  // sequence keeps raw pointers into the arena of its time (work counters, partial sums, the wait
  // verdict), and must find them intact however much the stream's scratch has grown since.
  char *retired[24];
  int n_retired;
  // Escape-time launches that their caller declared independent of their predecessors may begin before those
  // end (k_escape.cu).  Length of the current run of such launches, counted from the last launch that was
  // ordered behind everything before it; 0: the next launch is ordered.  Every other operation on the stream
  // that the library sees sets it back to 0.
  int escape_chain;
};

struct vrhi_sequence_t {
  vrhi_device_t *dev;
  cudaGraphExec_t exec;
  uint64_t kernels, retargets, rebuilds;
};

struct vrhi_event_t {
  vrhi_device_t *dev;
  cudaEvent_t e;
};

namespace vrhi {

constexpr size_t kCtrlBytes = 256;
// control-word indices (uint32) inside the arena's control block
enum { CTRL_STATUS = 0, CTRL_WORK0 = 1, CTRL_WORK1 = 2, CTRL_DONE = 3, CTRL_WAIT_OK = 4,
       CTRL_ESCAPE_RING = 8 /* 8 work counters, one per launch of a run of overlapping escape-time launches */ };

int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

#define VRHI_CUDA(call)                                                                   \
  do {                                                                                    \
    cudaError_t e__ = (call);                                                             \
    if (e__ != cudaSuccess)                                                               \
      return ::vrhi::fail(e__ == cudaErrorMemoryAllocation ? VRHI_ERR_OOM : VRHI_ERR_CUDA, \
                          "%s failed: %s", #call, cudaGetErrorString(e__));               \
  } while (0)

#define VRHI_TRY(expr)            \
  do {                            \
    int rc__ = (expr);            \
    if (rc__ != VRHI_OK) return rc__; \
  } while (0)

// Ensure the stream's arena holds `payload` bytes; returns control block and payload pointers.
int stream_arena(vrhi_stream_t *st, size_t payload, uint32_t **ctrl, char **payload_ptr);

struct ArgView {
  char *ptr;
  uint64_t bytes;
  int cls;       // class the caller declared for this use
  int buf_cls;   // class the buffer was created with
};

inline bool writable(const ArgView &a) {
  return a.buf_cls != VRHI_INPUT && a.buf_cls != VRHI_UNIFORM && a.buf_cls != VRHI_UNIFORM_CONSTANT;
}

typedef int (*LaunchFn)(vrhi_stream_t *st, const ArgView *args, int n_args, const void *params,
                        size_t params_size);

struct OpDef {
  const char *name;
  const char *signature;
  LaunchFn launch;
};

// Operator launchers, one per kernel family (defined in the k_*.cu files).
int launch_escape_time(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_fused_map(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_map_tape(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_row_sum(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_row_max(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_row_softmax(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_row_stats_softmax(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_col_sum(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_mse_tanh_fwd(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_mse_tanh_bwd(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_fp32_probe(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_vertex_transform(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_flat_color(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_widen_rows_u16(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_widen_rows_u8(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_gather_signal(vrhi_stream_t *, const ArgView *, int, const void *, size_t);
int launch_gather_pull_u16(vrhi_stream_t *, const ArgView *, int, const void *, size_t);

// Pieces of the image gather and of the small all-reduce (k_gather.cu), used by vrhi_group.cu.
int widen_rows_u16(vrhi_stream_t *st, const uint16_t *wire, uint32_t *image, const vrhi_widen_params &q, const uint32_t *ok);
int gather_push_u16(vrhi_stream_t *st, uint16_t *const *peer_wires, uint32_t n_peers, const uint16_t *wire, const vrhi_gather_params &q);
int widen_rows_squeezed(vrhi_stream_t *st, const uint8_t *bytes, const uint16_t *const *wire_by_rank, uint32_t *image, const vrhi_widen_params &q, const uint32_t *ok);
int gather_signal(vrhi_stream_t *st, uint32_t *const *peer_flags, uint32_t n, uint32_t slot, uint32_t seq);
int gather_wait(vrhi_stream_t *st, const uint32_t *flags, uint32_t world, uint32_t rank, uint32_t seq, uint32_t wait_ms, const uint32_t **ok);
int box_scatter(vrhi_stream_t *st, float *const *boxes, uint32_t world, uint32_t rank, const float *src, uint32_t n, uint32_t capacity);
int box_sum(vrhi_stream_t *st, const float *box, const uint32_t *ok, uint32_t world, float *dst, uint32_t n, uint32_t capacity);

// Operand count of a tape operation (vrhi_tape_op).
inline int tape_arity(int op) {
  switch (op) {
    case VRHI_T_CONST: return 0;
    case VRHI_T_ADD: case VRHI_T_SUB: case VRHI_T_MUL: case VRHI_T_DIV: case VRHI_T_MAX: case VRHI_T_MIN: case VRHI_T_EQ: return 2;
    case VRHI_T_FMA: return 3;
    default: return 1;
  }
}

// Run-time compiled tapes (tape_jit.cpp).  tape_jit_launch returns VRHI_OK (launched), 1 (leave it to
// the interpreter) or an error code.
int tape_jit_launch(vrhi_stream_t *st, const vrhi_tape_params &q, const float *const *in, float *const *out);
bool tape_jit_available();
int col_finalize(vrhi_stream_t *st, const float *partial, float *out, uint32_t groups, uint64_t cols, float scale);
void tape_jit_counters(uint64_t *compiled, uint64_t *launches, int *compiler_version, int *built_version);
std::string tape_jit_source(const vrhi_tape_params &q);

// Copies a caller's parameter block into a zero-initialised struct of the current layout,
// honouring the leading size field (older, shorter callers leave new fields zero).
template <class P>
int read_params(const void *params, size_t params_size, P *out) {
  *out = P{};
  if (!params || params_size < sizeof(uint32_t)) return fail(VRHI_ERR_INVALID, "missing parameter block");
  uint32_t declared = *static_cast<const uint32_t *>(params);
  if (declared > params_size) return fail(VRHI_ERR_SIZE, "parameter block declares %u bytes but %zu were passed", declared, params_size);
  size_t n = declared < sizeof(P) ? declared : sizeof(P);
  memcpy(out, params, n);
  return VRHI_OK;
}

// An integer from the environment, or `fallback` when the variable is unset or outside [lo, hi].  The
// tuning and behaviour switches of this library are read ONCE per process, by callers of the form
//   static const int v = env_int("NAME", lo, hi, fallback);
// so that nothing on a launch path calls getenv.
inline int env_int(const char *name, int lo, int hi, int fallback) {
  const char *e = getenv(name);
  if (!e || !*e) return fallback;
  const int v = atoi(e);
  return v >= lo && v <= hi ? v : fallback;
}

// rows * cols as an element count, refused (VRHI_ERR_SIZE) beyond 2^40 elements: checked before any
// byte count is formed, so that a product that wraps in 64 bits can never pass a size check.
inline int element_count(uint64_t rows, uint64_t cols, const char *name, uint64_t *out) {
  constexpr uint64_t kMax = 1ull << 40;
  if (rows != 0 && cols > kMax / rows) return fail(VRHI_ERR_SIZE, "%s: %llu x %llu elements are out of range (at most 2^40)", name, (unsigned long long)rows, (unsigned long long)cols);
  *out = rows * cols;
  return VRHI_OK;
}

inline int post_launch(vrhi_stream_t *st, const char *what, int kernels = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(VRHI_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  st->launches += (uint64_t)kernels;
  st->escape_chain = 0;  // the escape-time launcher sets its own value after this
  return VRHI_OK;
}

}  // namespace vrhi
