/*
 * vrhi.h -- C ABI of libvrhi.so, the B200 (sm_100a) execution backend for VernonDSL-style
 * data-parallel kernels: the per-element escape-time map of fractal.py, fused elementwise map
 * chains, the row reductions and softmax they feed, and the backward of those operators.
 *
 * WHAT THIS BOUNDARY REPLACES.  The reference project has no runtime, device layer, operator
 * registry or FFI of its own; nothing in its tree calls a kernel library.  Its only executable
 * statement of the path is fractal.py, which reaches a GPU through the third-party Taichi
 * runtime (fractal.py:5 ti.init, :8 ti.field, :16 @ti.kernel, :31 paint(t)).  The entry points
 * below are therefore what a Vernon runtime would bind in place of those Taichi calls; each
 * group names the reference line it stands in for.  The one Vernon-specific artefact that
 * constrains this ABI is the `vernon.semantic` argument vocabulary
 * (source/lib/Dialect/Vernon/Transforms/VernonToSpirv.cpp:38-56,
 * source/tests/integration/color.mlir:4-9,43-45), kept here as `vrhi_arg_class`.
 *
 * RULES.  C linkage, plain pointers and sizes, opaque handles; no C++ or torch types.  Every
 * function returns an int status (0 = VRHI_OK, negative = VRHI_ERR_*); `vrhi_last_error()`
 * returns a thread-local message for the last failure on the calling thread.  Nothing aborts,
 * exits or traps.  There is NO CPU fallback: a shape or mode a kernel does not support returns
 * VRHI_ERR_UNSUPPORTED.  Handles are not locked internally: drive one stream from one thread
 * at a time; different streams and devices may be driven from different threads.
 */
#ifndef VRHI_H_
#define VRHI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define VRHI_API __attribute__((visibility("default")))
#else
#define VRHI_API
#endif

#define VRHI_VERSION 100 /* major*100 + minor */

/* ---------------------------------------------------------------- status codes ---------- */
enum vrhi_status {
  VRHI_OK = 0,
  VRHI_ERR_INVALID = -1,     /* NULL handle, bad enum, bad argument count ...                 */
  VRHI_ERR_CUDA = -2,        /* a CUDA runtime call failed; message holds cudaGetErrorString  */
  VRHI_ERR_OOM = -3,         /* device or pinned-host allocation failed                       */
  VRHI_ERR_UNSUPPORTED = -4, /* shape / mode not implemented by any kernel (no CPU fallback)  */
  VRHI_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up                            */
  VRHI_ERR_NOT_FOUND = -6,   /* unknown operator or semantic name                             */
  VRHI_ERR_SIZE = -7,        /* buffer too small / size mismatch / misaligned offset          */
  VRHI_ERR_GRAPH = -8,       /* execution-graph construction or compilation error            */
  VRHI_ERR_PEER = -9         /* another rank's memory could not be mapped, or the caller's all-gather failed */
};

/* Thread-local text of the last error on this thread ("" if none).  Never NULL. */
VRHI_API const char *vrhi_last_error(void);
VRHI_API int vrhi_version(void);

/* ------------------------------------------------------------- argument classes --------- */
/* The `vernon.semantic` vocabulary: VernonToSpirv.cpp:44-55 (input, output, uniform,
 * uniform_constant, storage_buffer, image) plus `varying`, which color.mlir:9,44 uses and the
 * reference pass leaves unhandled.  A buffer is created with one class; operators check that
 * what they write is not INPUT / UNIFORM / UNIFORM_CONSTANT. */
enum vrhi_arg_class {
  VRHI_INPUT = 0,
  VRHI_OUTPUT = 1,
  VRHI_UNIFORM = 2,
  VRHI_UNIFORM_CONSTANT = 3,
  VRHI_STORAGE_BUFFER = 4,
  VRHI_IMAGE = 5,
  VRHI_VARYING = 6
};
/* "input" -> VRHI_INPUT ...; VRHI_ERR_NOT_FOUND for any other string. */
VRHI_API int vrhi_arg_class_from_semantic(const char *semantic, int *out_class);
VRHI_API const char *vrhi_arg_class_name(int arg_class); /* NULL if out of range */

/* ------------------------------------------------------------------- handles ------------ */
typedef struct vrhi_device_t *vrhi_device;
typedef struct vrhi_buffer_t *vrhi_buffer;
typedef struct vrhi_stream_t *vrhi_stream;
typedef struct vrhi_event_t *vrhi_event;
typedef struct vrhi_graph_t *vrhi_graph;
typedef struct vrhi_sequence_t *vrhi_sequence;
typedef struct vrhi_group_t *vrhi_group;
typedef struct vrhi_exchange_t *vrhi_exchange;

/* ------------------------------------------------------------------- device ------------- */
/* Stands in for fractal.py:5 (ti.init(arch=...)): choose and open the compute device. */
typedef struct vrhi_device_props {
  uint32_t size;           /* set to sizeof(vrhi_device_props) by the caller */
  int32_t ordinal;
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  int32_t sm_clock_khz;    /* maximum SM clock */
  int32_t mem_clock_khz;
  int32_t l2_bytes;
  int32_t smem_per_block_optin;
  uint64_t total_mem_bytes;
  char name[128];
} vrhi_device_props;

VRHI_API int vrhi_device_count(int *out_count);
VRHI_API int vrhi_device_create(int ordinal, vrhi_device *out_dev);
VRHI_API int vrhi_device_destroy(vrhi_device dev); /* NULL is accepted */
VRHI_API int vrhi_device_props_get(vrhi_device dev, vrhi_device_props *out_props);
VRHI_API int vrhi_device_synchronize(vrhi_device dev);
/* Test hook for the out-of-memory path: refuse allocations once more than `bytes` are held by
 * this device handle (0 = no limit).  Host-side accounting only. */
VRHI_API int vrhi_device_set_alloc_limit(vrhi_device dev, uint64_t bytes);
VRHI_API int vrhi_device_allocated(vrhi_device dev, uint64_t *out_bytes);

/* ------------------------------------------------------------------- buffers ------------ */
/* Stands in for fractal.py:8 (ti.field(dtype, shape)): dense device storage.  The library owns
 * device memory it creates; the caller owns host memory and any pointer it wraps. */
VRHI_API int vrhi_buffer_create(vrhi_device dev, uint64_t bytes, int arg_class, vrhi_buffer *out_buf);
/* Adopt device memory owned by someone else (for example a torch tensor's data_ptr). */
VRHI_API int vrhi_buffer_wrap(vrhi_device dev, void *device_ptr, uint64_t bytes, int arg_class,
                              vrhi_buffer *out_buf);
VRHI_API int vrhi_buffer_destroy(vrhi_buffer buf); /* NULL is accepted */
VRHI_API int vrhi_buffer_size(vrhi_buffer buf, uint64_t *out_bytes);
VRHI_API int vrhi_buffer_class(vrhi_buffer buf, int *out_class);
VRHI_API int vrhi_buffer_device_ptr(vrhi_buffer buf, void **out_ptr);
/* Asynchronous on `stream` (NULL = the device's default stream, then synchronous).  Host memory
 * should be pinned (vrhi_host_alloc) for the copy to overlap. */
VRHI_API int vrhi_buffer_upload(vrhi_buffer buf, uint64_t offset, const void *host, uint64_t bytes,
                                vrhi_stream stream);
VRHI_API int vrhi_buffer_download(vrhi_buffer buf, uint64_t offset, void *host, uint64_t bytes,
                                  vrhi_stream stream);
VRHI_API int vrhi_buffer_fill_u8(vrhi_buffer buf, uint64_t offset, int value, uint64_t bytes,
                                 vrhi_stream stream);
VRHI_API int vrhi_host_alloc(uint64_t bytes, void **out_host); /* pinned */
VRHI_API int vrhi_host_free(void *host);
/* Device-to-device copy of `rows` runs of `width_bytes` bytes (pitches in bytes; rows = 1 is a
 * plain copy).  Source and destination may live on different GPUs of one box, including a
 * destination opened with vrhi_buffer_ipc_open: the copy engines move the data over NVLink
 * without occupying SMs, so it overlaps kernels on other streams. */
VRHI_API int vrhi_buffer_copy_2d(vrhi_buffer dst, uint64_t dst_offset, uint64_t dst_pitch, vrhi_buffer src,
                                 uint64_t src_offset, uint64_t src_pitch, uint64_t width_bytes, uint64_t rows,
                                 vrhi_stream stream);
/* Multi-process sharing inside one box (one process per GPU): export a 64-byte handle of a buffer
 * this library allocated, and open another process's handle as a buffer that can be a copy
 * destination.  Destroying an opened buffer closes the mapping, not the memory. */
#define VRHI_IPC_HANDLE_BYTES 64
VRHI_API int vrhi_buffer_ipc_export(vrhi_buffer buf, void *out_handle /* VRHI_IPC_HANDLE_BYTES */);
VRHI_API int vrhi_buffer_ipc_open(vrhi_device dev, const void *handle, uint64_t bytes, int arg_class,
                                  vrhi_buffer *out_buf);

/* ---------------------------------------------------------------- streams / events ------ */
VRHI_API int vrhi_stream_create(vrhi_device dev, vrhi_stream *out_stream);
/* Adopt an existing CUDA stream handle (a cudaStream_t / CUstream, e.g. torch's). */
VRHI_API int vrhi_stream_wrap(vrhi_device dev, void *cuda_stream, vrhi_stream *out_stream);
VRHI_API int vrhi_stream_destroy(vrhi_stream stream); /* NULL is accepted */
VRHI_API int vrhi_stream_synchronize(vrhi_stream stream);
/* Device-side status word of the stream: kernels with bounded waits or index checks record a
 * VRHI_ERR_* there instead of trapping.  Synchronises the stream, returns and clears it. */
VRHI_API int vrhi_stream_check(vrhi_stream stream);
/* Number of kernels this library has launched on the stream since it was created. */
VRHI_API int vrhi_stream_launch_count(vrhi_stream stream, uint64_t *out_count);
VRHI_API int vrhi_event_create(vrhi_device dev, vrhi_event *out_event);
VRHI_API int vrhi_event_destroy(vrhi_event event); /* NULL is accepted */
VRHI_API int vrhi_event_record(vrhi_event event, vrhi_stream stream);
VRHI_API int vrhi_event_synchronize(vrhi_event event);
VRHI_API int vrhi_event_elapsed_ms(vrhi_event start, vrhi_event stop, float *out_ms);
VRHI_API int vrhi_stream_wait_event(vrhi_stream stream, vrhi_event event);

/* ---- recorded launch sequences ------------------------------------------------------------
 * The frame loop of fractal.py:30-33 relaunches one kernel with a new uniform per frame.  For
 * small frames the cost of a frame is the launch, not the arithmetic, so a run of frames is
 * recorded once and replayed as one CUDA graph launch.
 *
 * vrhi_sequence_begin puts the stream into recording: every vrhi_op_launch, vrhi_graph_launch,
 * vrhi_buffer_fill and device-to-device copy issued on it until vrhi_sequence_end is recorded
 * instead of executed.  Uniforms are part of what is recorded.  vrhi_sequence_end with
 * *inout_seq == NULL builds a new sequence; with an existing sequence it re-targets that
 * sequence in place (same launches, new uniforms or buffers: no rebuild) and rebuilds only when the
 * shape of the recording changed.  Each operator must have run once on the stream before it is
 * recorded (its scratch is sized then; nothing may be allocated while recording, and a
 * launch that would need to allocate returns VRHI_ERR_INVALID).  Host transfers and
 * synchronisation are not recordable.
 * Reference counterpart: none; fractal.py leaves launching to its runtime. */
VRHI_API int vrhi_sequence_begin(vrhi_stream stream);
/* Draw a second stream into the recording of `stream`: what is launched on `side` from here on is
 * recorded too, ordered behind everything recorded on `stream` so far and otherwise free to run
 * beside it (frames k and k+1 of a frame loop on alternating streams overlap: the last blocks of
 * one frame drain while the first of the next start).  At most 4 side streams; they rejoin at
 * vrhi_sequence_end, which must be called on `stream`. */
VRHI_API int vrhi_sequence_fork(vrhi_stream stream, vrhi_stream side);
VRHI_API int vrhi_sequence_end(vrhi_stream stream, vrhi_sequence *inout_seq);
VRHI_API int vrhi_sequence_launch(vrhi_sequence seq, vrhi_stream stream);
/* kernels per replay, times the sequence was re-targeted in place, times it was rebuilt */
VRHI_API int vrhi_sequence_stats(vrhi_sequence seq, uint64_t *out_kernels, uint64_t *out_retargets, uint64_t *out_rebuilds);
VRHI_API int vrhi_sequence_destroy(vrhi_sequence seq); /* NULL is accepted */

/* ------------------------------------------------------------------ operators ----------- */
/* Stands in for fractal.py:16,31 (@ti.kernel definition and its launch): a registry of named
 * kernels, each launched with buffer arguments and a small POD parameter block ("uniforms").
 * The registry is immutable after library load. */
typedef struct vrhi_arg {
  vrhi_buffer buffer;
  uint64_t offset;   /* byte offset into the buffer; must be a multiple of 16 */
  uint64_t bytes;    /* bytes of the view; 0 = from offset to the end of the buffer */
  int32_t arg_class; /* how this operator uses the view (checked against the op's signature) */
  int32_t reserved;
} vrhi_arg;

VRHI_API int vrhi_op_count(int *out_count);
VRHI_API int vrhi_op_name(int op, const char **out_name);
VRHI_API int vrhi_op_lookup(const char *name, int *out_op);
/* One line describing the op's arguments and parameter struct, for diagnostics. */
VRHI_API int vrhi_op_signature(int op, const char **out_text);
VRHI_API int vrhi_op_launch(vrhi_stream stream, int op, const vrhi_arg *args, int n_args,
                            const void *params, size_t params_size);

/* Every parameter struct starts with its own size so that it can grow compatibly. */

/* op "escape_time" -- args: [0] OUTPUT/IMAGE image, row-major [height][width].
 * Per pixel (i, j): x = x0 + (float)i*dx, y = y0 + (float)j*dy (pixel corner, fractal.py:20);
 * MANDELBROT: z = 0, c = (x, y);  JULIA: z = (x, y), c = (cr, ci).
 * Loop (fractal.py:21-24): a = zr*zr; b = zi*zi; stop if test(a+b) or count == max_iter;
 * t = zr*zi; zi = (t+t)+ci; zr = (a-b)+cr; ++count.
 * EXACT mode performs exactly these binary32 roundings (no contraction across them), so the
 * counts are reproducible bit for bit; FAST mode lets multiply-adds fuse and may differ on a
 * small fraction of pixels.
 * Rows processed: chunks k = chunk_first, chunk_first+chunk_step, ... (chunk_count of them),
 * chunk k covering rows [k*chunk_rows, min(height, (k+1)*chunk_rows)).  Results are written at
 * their true position in the full image.  chunk_rows = 0 means "the whole image". */
enum { VRHI_ESCAPE_MANDELBROT = 0, VRHI_ESCAPE_JULIA = 1 };
enum { VRHI_ESCAPE_EXACT = 0, VRHI_ESCAPE_FAST = 1 };
enum { VRHI_TEST_NORM2_GT = 0, /* stop when a+b > bound                         */
       VRHI_TEST_NORM_GE = 1   /* stop unless sqrtf(a+b) < bound (fractal.py:22) */ };
enum { VRHI_OUT_COUNT_U32 = 0, VRHI_OUT_COUNT_U16 = 1,
       VRHI_OUT_COLOR_F32 = 2 /* 1 - count*color_scale, fractal.py:25 */ };
typedef struct vrhi_escape_params {
  uint32_t size;
  uint32_t kind, mode, test, output;
  uint32_t width, height;
  uint32_t max_iter;
  float x0, y0, dx, dy;
  float cr, ci;
  float bound;
  float color_scale;
  uint32_t chunk_rows, chunk_first, chunk_step, chunk_count;
  uint32_t flags; /* VRHI_ESCAPE_FLAG_* */
} vrhi_escape_params;
/* Run the kernel that tests on every step even where the faster regrouping kernel applies
 * (exact mode, NORM2_GT with bound >= 4, |c| <= 1.5).  Results are identical either way. */
#define VRHI_ESCAPE_FLAG_CHECKED_ONLY 1u
/* The real axis runs along the rows and the imaginary axis along the columns: pixel (row j,
 * column i) has real part y0 + j*dy and imaginary part x0 + i*dx.  This is the memory order of a
 * field indexed [i, j] whose first index feeds the real part (fractal.py:8,20). */
#define VRHI_ESCAPE_FLAG_TRANSPOSED 2u
/* Bits 8-10, k = 1..7: the caller declares that this launch reads and writes nothing that the k
 * escape_time launches before it on the same stream write (frames that go round a ring of k+1
 * images, as the loop of fractal.py:30-33 would with a swap chain).  Such a launch may begin while
 * those launches still run, so that its first blocks fill the SMs the last blocks of the frame
 * before leave idle; it never completes before them, and whatever else follows on the stream
 * (copies, events, other operators, launches without the declaration) is ordered behind all of
 * them as usual.  k = 0 (the default): the launch is ordered behind everything before it.
 * Results are the same either way. */
#define VRHI_ESCAPE_FLAG_INDEPENDENT_SHIFT 8
#define VRHI_ESCAPE_FLAG_INDEPENDENT_MASK 0x700u
#define VRHI_ESCAPE_INDEPENDENT_OF(k) (((uint32_t)(k) & 7u) << VRHI_ESCAPE_FLAG_INDEPENDENT_SHIFT)

/* op "escape_time", optional second argument: a uint16 image of the same [height][width]
 * geometry that receives every count a second time (uint32 counts only, max_iter <= 65535).
 * It is the form in which a rank sends its rows to its peers when the image is gathered over
 * NVLink: half the bytes, nothing lost.  Optional third argument: a plane of bytes of the same
 * geometry that receives min(count, 255): a quarter of the bytes; a byte of 255 sends the reader
 * to the uint16 image (vrhi_exchange_* moves this plane where it pays and fetches the rest).
 *
 * op "widen_rows_u16" -- the receiving side: copies uint16 counts into the uint32 image for the
 * rows of slabs slab_first .. slab_first+slab_count-1 (a slab = `world` consecutive chunks of
 * chunk_rows rows), leaving out the chunks of `skip_rank` (the caller's own, already present in
 * full width); skip_rank >= world widens every chunk.
 * args: [0] wire (uint16 [height][width]), [1] image (uint32 [height][width], writable).
 * op "widen_rows_u8" -- the same from a plane of bytes min(count, 255): args [0] bytes (uint8
 * [height][width]), [1] image, [2..] the uint16 wire images of ranks 0..world-1 (mapped peer memory
 * or local); a 16-pixel granule that shows a byte of 255 is taken from the wire image of the rank
 * that owns the row.  width a multiple of 16.
 * Reference counterpart: none (the reference runs on one device). */
typedef struct vrhi_widen_params {
  uint32_t size;
  uint32_t width, height;
  uint32_t chunk_rows, world, skip_rank;
  uint32_t slab_first, slab_count;
  uint32_t slab_stride; /* slabs slab_first + k*slab_stride, k < slab_count; 0 reads as 1 */
} vrhi_widen_params;

/* ops "gather_signal" and "gather_pull_u16" -- the gather in pull form, for ranks whose
 * buffers are mapped into one another (vrhi_buffer_ipc_export/open): transfer over NVLink and
 * widening are one kernel on the receiving side.
 * gather_signal: args = the flag arrays (uint32[world], zero-initialised, one per rank) of the
 *   world-1 peers, in any order; stores `seq` into slot `rank` of each.  Launch it on the stream
 *   that computed the rows, after them.
 * gather_pull_u16: args = [0] the caller's own flag array, [1] its uint32 image, [2..] the uint16
 *   wire images of ranks 0..world-1 without the caller's own, in rank order.  Waits until every
 *   peer's slot in the flag array has reached `seq` (a one-warp kernel; at most wait_ms
 *   milliseconds, default 2000; on expiry nothing is copied and vrhi_stream_check returns
 *   VRHI_ERR_TIMEOUT), then copies the peers' rows of the given slabs into the image.
 * Sequence numbers must grow by less than 2^31 between a wait and the value it waits for.
 * A rank must not overwrite rows a peer may still be pulling: alternate two wire images.
 * Reference counterpart: none (the reference runs on one device). */
#define VRHI_GATHER_MAX_WORLD 8
typedef struct vrhi_gather_params {
  uint32_t size;
  uint32_t width, height;
  uint32_t chunk_rows, world, rank;
  uint32_t slab_first, slab_count;
  uint32_t seq;
  uint32_t wait_ms;
  uint32_t slab_stride; /* as in vrhi_widen_params */
} vrhi_gather_params;

/* op "fused_map" -- the map chain  out = tanh(a*x + y) * exp(-0.5*x*x) + sqrt(|y| + 1e-3)
 * as one kernel.  args: [0] a, [1] x, [2] y (INPUT, n floats), [3] out (OUTPUT, n floats). */
typedef struct vrhi_map_params {
  uint32_t size;
  uint32_t reserved;
  uint64_t n;
} vrhi_map_params;

/* op "map_tape" -- a fused chain of elementwise operations given as a register tape, run as
 * one kernel.  args: n_inputs INPUT views then n_outputs OUTPUT views.  Input k is a full
 * [rows][cols] array unless bit k is set in one of the masks: row_vector_mask = a [cols] row
 * vector broadcast down the rows; col_vector_mask = a [rows] vector, one value per row,
 * broadcast along it; scalar_mask = a single float broadcast everywhere.
 * Instruction t computes value (n_inputs + t) from earlier values. */
enum vrhi_tape_op {
  VRHI_T_CONST = 0, /* imm */
  VRHI_T_ADD, VRHI_T_SUB, VRHI_T_MUL, VRHI_T_DIV, VRHI_T_MAX, VRHI_T_MIN,  /* a, b */
  VRHI_T_FMA,                                                           /* a*b + c */
  VRHI_T_NEG, VRHI_T_ABS, VRHI_T_SQUARE, VRHI_T_SQRT, VRHI_T_RSQRT, VRHI_T_RECIP,
  VRHI_T_EXP, VRHI_T_LOG, VRHI_T_TANH, VRHI_T_SIGMOID, VRHI_T_RELU, VRHI_T_COS, VRHI_T_SIN,
  VRHI_T_SIGN, VRHI_T_STEP, /* step: 1 if a > 0 else 0 */
  VRHI_T_EQ,                /* 1 if a == b else 0 */
  VRHI_T_OPCOUNT
};
#define VRHI_TAPE_MAX_INSTR 64
#define VRHI_TAPE_MAX_INPUTS 8
#define VRHI_TAPE_MAX_OUTPUTS 4
typedef struct vrhi_tape_instr {
  uint16_t op;
  uint16_t a, b, c; /* value indices */
  float imm;
} vrhi_tape_instr;
typedef struct vrhi_tape_params {
  uint32_t size;
  uint32_t n_inputs, n_outputs, n_instr;
  uint64_t rows, cols;              /* element count = rows*cols */
  uint32_t row_vector_mask, col_vector_mask, scalar_mask;
  uint32_t out_value[VRHI_TAPE_MAX_OUTPUTS]; /* value index stored to output k */
  vrhi_tape_instr instr[VRHI_TAPE_MAX_INSTR];
  uint32_t flags; /* VRHI_TAPE_FLAG_* */
  uint32_t colsum_mask; /* bit k: output k is not stored; its column sums are: the argument is a [cols] array.
                           Needs the compiled path (VRHI_ERR_UNSUPPORTED otherwise). Deterministic: fixed order. */
} vrhi_tape_params;
/* A tape normally runs as a kernel compiled for it at first use (NVRTC, cached; values in
 * registers, HBM-bound).  This flag, or VRHI_TAPE_JIT=0 in the environment, selects the
 * interpreting kernel instead, which is also what runs where NVRTC is not installed, for column
 * counts that are not a multiple of 4 and for unaligned arrays.  Both give the same bits. */
#define VRHI_TAPE_FLAG_INTERPRET 1u
/* Tapes compiled so far in this process, launches of compiled tapes, the version of the run-time
 * compiler in use (major*1000 + minor*10; 0 before the first tape, or when there is none) and the
 * CUDA version the library was built with, counted the same way.  When the two versions are equal
 * the compiled and the interpreting kernel give the same bits; with another compiler version the
 * transcendental functions may round differently in the last place.  Any pointer may be NULL. */
VRHI_API int vrhi_tape_jit_stats(uint64_t *out_compiled, uint64_t *out_launches, int *out_compiler_version, int *out_built_version);
/* The CUDA source generated for a tape (NUL-terminated, truncated to `capacity`); *out_needed
 * receives the full length including the terminator.  Needs no device. */
VRHI_API int vrhi_tape_source(const vrhi_tape_params *params, char *buffer, uint64_t capacity, uint64_t *out_needed);

/* ops "row_sum", "row_max": args [0] INPUT [rows][cols] floats, [1] OUTPUT [rows] floats.
 * op "row_softmax": args [0] INPUT [rows][cols], [1] OUTPUT [rows][cols]; max is subtracted.
 * op "row_stats_softmax": one pass producing all three: args [0] INPUT, [1] OUTPUT sum[rows],
 *   [2] OUTPUT max[rows], [3] OUTPUT softmax[rows][cols].
 * op "col_sum": args [0] INPUT [rows][cols], [1] OUTPUT [cols]. Deterministic (no float atomics). */
typedef struct vrhi_rows_params {
  uint32_t size;
  uint32_t reserved;
  uint64_t rows, cols;
} vrhi_rows_params;

/* op "mse_tanh_fwd": loss contribution of `rows` rows:  sum((tanh(W*x + b[col]) - t)^2) / denom.
 *   args [0] W, [1] x, [2] b ([cols]), [3] t (INPUT), [4] OUTPUT loss (one float).
 * op "mse_tanh_bwd": g = 2*(y - t)*(1 - y*y)/denom with y recomputed; dW = g*x, dx = g*W,
 *   db[col] = sum over rows of g (fixed summation order, bit-reproducible).
 *   args [0] W, [1] x, [2] b, [3] t (INPUT), [4] dW, [5] dx, [6] db (OUTPUT),
 *   optional [7] OUTPUT loss (one float).
 * denom = 0 means rows*cols; a row shard of a larger matrix passes the whole element count. */
typedef struct vrhi_mse_params {
  uint32_t size;
  uint32_t reserved;
  uint64_t rows, cols;
  double denom;
} vrhi_mse_params;

/* ops "vertex_transform" and "flat_color": the arithmetic of the reference's shader input
 * (source/tests/integration/color.mlir) over arrays, no graphics API involved; both take
 * vrhi_map_params with n = number of vertices / fragments.
 *   vertex_transform (color.mlir:4-39): args [0] pos INPUT f32[n][3], [1] model, [2] view,
 *     [3] proj UNIFORM f32[16] row-major, [4] gl_position OUTPUT f32[n][4] =
 *     proj*(view*(model*(p0,p1,p2,1))), [5] varying VARYING f32[n][3] = pos.
 *   flat_color (color.mlir:43-59): args [0] color UNIFORM f32[3], [1] fragments IMAGE f32[n][4],
 *     every fragment = (c0,c1,c2,1). */

/* op "fp32_probe": dependent-free fma chains, for measuring the FP32 issue peak the escape-time
 * kernel is bounded by.  args [0] OUTPUT (>= 4 bytes).  Executes `ffma_per_thread` fma instructions
 * in each of `threads` threads.  variant 0: scalar fma.rn.f32 (the roofline's denominator);
 * 1: packed fma.rn.f32x2, two lane-FMAs per instruction; 2: packed with one integer add per fma;
 * 3: scalar with one integer add per fma. */
typedef struct vrhi_probe_params {
  uint32_t size;
  uint32_t variant;
  uint64_t ffma_per_thread;
  uint64_t threads; /* 0 = fill the device */
} vrhi_probe_params;

/* Column sums without any allocation (no counterpart in the reference).
 * For callers that cannot afford or are not allowed an allocation at call time: latency-bound
 * frame or control loops, processes whose device memory was divided up front, code that must
 * leave the allocator untouched.  out[c] = sum over rows of in[r][c], row-major floats, the same
 * deterministic two-stage algorithm as the "col_sum" operator, but the per-row-group partial
 * sums live in a fixed 1 MiB array inside the library image (every GPU that loads the library
 * holds it until the process exits) instead of the stream arena.  Takes raw device pointers and
 * a raw CUDA stream handle (NULL = default stream); works on the current device.
 * Limits: cols <= 262144 (VRHI_ERR_SIZE beyond that); `in` 16-byte aligned.
 * The first call on a device looks up the array's device address; make that first call before
 * any stream capture begins.  All calls share the one array: calls whose kernels could overlap
 * on the GPU (different streams without an ordering between them) race on it.  Nothing in the
 * array needs clearing: each call writes every partial it later reads. */
VRHI_API int vrhi_col_sum_static_scratch(const float *in_device, float *out_device, uint64_t rows,
                                         uint64_t cols, void *cuda_stream);

/* --------------------------------------------------------------- partitioning ----------- */
/* Host-side planning for N devices in one box, one process per device.  No CUDA calls. */
enum { VRHI_PART_CONTIGUOUS = 0, VRHI_PART_CYCLIC = 1 };
typedef struct vrhi_row_partition {
  uint32_t chunk_rows, chunk_first, chunk_step, chunk_count; /* feed vrhi_escape_params */
  uint64_t rows_owned;
} vrhi_row_partition;
/* Split `total_rows` image rows over `world` ranks.  CONTIGUOUS: one band per rank (sizes
 * differ by at most one chunk).  CYCLIC: chunks of `chunk_rows` rows dealt round-robin, which
 * balances escape-time work whose cost varies smoothly over the image. */
VRHI_API int vrhi_partition_rows(uint64_t total_rows, uint32_t chunk_rows, uint32_t world,
                                 uint32_t rank, int scheme, vrhi_row_partition *out);
/* Split `n` leading-axis units evenly (first n%world ranks get one more). */
VRHI_API int vrhi_partition_leading(uint64_t n, uint32_t world, uint32_t rank, uint64_t *out_begin,
                                    uint64_t *out_count);

/* ------------------------------------------------------------- groups of GPUs ----------- */
/* N GPUs of one box, one rank per GPU; a rank is a process, or a thread of a process that drives
 * several GPUs.  The reference runs on one device (fractal.py:5): none of this has a counterpart
 * there.  The library brings no network layer and no collective library: to learn of each other's
 * buffers the ranks need ONE service from the caller, an all-gather of small byte records (MPI,
 * a key-value store, pipes, shared memory ...), used only while a group or an exchange is being
 * created.  Everything after that is kernels of this library storing into mapped peer memory over
 * NVLink and sequence numbers in flag arrays; each device-side wait is one warp with a time limit
 * (default 2 s) that records VRHI_ERR_TIMEOUT in a status word instead of hanging.
 *
 * vrhi_allgather_fn: `send` holds `bytes` bytes of this rank; on return `recv` holds world*bytes
 * bytes, rank r's record at offset r*bytes.  Returns 0 on success.  Every rank calls the creating
 * (and destroying) functions in the same order, so the all-gathers match up; it should carry a time
 * limit of its own, because a rank whose creation fails half way (VRHI_ERR_PEER: a peer's memory
 * cannot be mapped) leaves the others waiting in it. */
typedef int (*vrhi_allgather_fn)(void *user, const void *send, void *recv, uint64_t bytes);
#define VRHI_GROUP_MAX_WORLD 8
VRHI_API int vrhi_group_create(vrhi_device dev, uint32_t world, uint32_t rank, vrhi_allgather_fn allgather, void *user,
                               vrhi_group *out_group);
/* Every rank calls it, once no rank uses the group any more: the ranks meet once inside (one round of
 * the all-gather), because a rank's memory must outlive the other ranks' mappings of it.  The same
 * holds for vrhi_exchange_destroy.  NULL is accepted. */
VRHI_API int vrhi_group_destroy(vrhi_group group);
VRHI_API int vrhi_group_info(vrhi_group group, uint32_t *out_world, uint32_t *out_rank);
VRHI_API int vrhi_group_set_wait_ms(vrhi_group group, uint32_t wait_ms); /* limit of the device-side waits; 0 = 2000 */
/* Sum of `n` floats (n <= 16384) at `offset` bytes of `buf` over all ranks, in place, enqueued on
 * `stream`: the db row and the loss of a row-sharded backward, partial reductions.  Every rank adds
 * the ranks' values in rank order: the same bits everywhere.  Calls of one rank must be ordered one
 * behind the other on the GPU (one stream, or streams that wait for each other), and every rank
 * makes the same calls in the same order.  A peer that does not arrive within the time limit
 * leaves `buf` untouched; vrhi_stream_check(stream) then returns VRHI_ERR_TIMEOUT. */
VRHI_API int vrhi_group_all_reduce_sum_f32(vrhi_group group, vrhi_buffer buf, uint64_t offset, uint64_t n, vrhi_stream stream);

/* Gather of an escape-time image whose row chunks are dealt to the ranks round-robin
 * (vrhi_partition_rows, VRHI_PART_CYCLIC): every rank ends every step with the whole uint32 image.
 * `image` is this rank's full-size image [height][width]; height must be a whole number of chunks
 * and the chunks must divide evenly over the ranks; width a multiple of 8.  Counts cross NVLink as
 * uint16 (max_iter <= 65535): the exchange owns two uint16 wire images per rank, which alternate
 * from step to step so that a fast rank never stores into rows a slower peer is still reading.
 *
 * From three ranks on the exchange by default squeezes the counts further: the kernel also writes a
 * plane of bytes min(count, 255) (a third argument), that plane is what the copy engines move, and
 * the receiving kernel fetches the 16-pixel granules that show a byte of 255 from the owner's uint16
 * wire image over NVLink.  Lossless whatever the image; VRHI_EXCHANGE_SQUEEZE=0/1 overrides.
 *
 * One step on every rank:
 *   vrhi_exchange_planes(ex, &wire, &bytes);           this step's wire image and byte plane (bytes == NULL: not squeezing)
 *   for each group of slabs (the same groups, in the same order, on every rank; a slab = `world`
 *   consecutive chunks, one per rank):
 *     vrhi_op_launch(compute_stream, escape_time, {image, wire[, bytes]}, params of the rank's chunks of the group);
 *     vrhi_exchange_publish(ex, compute_stream, slab_first, slab_count, slab_stride);
 *   vrhi_exchange_complete(ex, stream);
 * publish marks the point of compute_stream behind which the rank's rows of those slabs are ready; it
 * costs one event record, so that the caller's next launch is not held up.  The transfer of every
 * published group is enqueued, in order, by the next call that is not a publish (complete or check;
 * after 16 groups at the latest): behind that point, on streams of the exchange, the copy engines send
 * the rank's rows into every peer's wire image (or byte plane) and the rank's sequence number is
 * raised there; on another stream a bounded wait for every peer's number is followed by the widening of
 * their rows into `image`.  complete makes `stream` wait for all of the step's arrivals and for this
 * rank's own transfers, and switches to the other wire image; work enqueued on `stream` afterwards
 * sees the whole image, and the next step's launches must be ordered behind it.  No host
 * synchronisation anywhere in a step.
 * vrhi_exchange_check synchronises the exchange's streams and returns VRHI_ERR_TIMEOUT if a peer
 * failed to arrive in time (its rows are then missing from the image). */
VRHI_API int vrhi_exchange_create(vrhi_group group, vrhi_buffer image, uint32_t width, uint32_t height, uint32_t chunk_rows,
                                  vrhi_exchange *out_exchange);
VRHI_API int vrhi_exchange_destroy(vrhi_exchange exchange); /* before the group; NULL is accepted */
VRHI_API int vrhi_exchange_planes(vrhi_exchange exchange, vrhi_buffer *out_wire, vrhi_buffer *out_bytes);
VRHI_API int vrhi_exchange_publish(vrhi_exchange exchange, vrhi_stream compute_stream, uint32_t slab_first,
                                   uint32_t slab_count, uint32_t slab_stride);
VRHI_API int vrhi_exchange_complete(vrhi_exchange exchange, vrhi_stream stream);
VRHI_API int vrhi_exchange_check(vrhi_exchange exchange);
/* Kernels the exchange has launched on its own streams so far. */
VRHI_API int vrhi_exchange_launch_count(vrhi_exchange exchange, uint64_t *out_count);

/* ------------------------------------------------------------- execution graph ---------- */
/* A small tensor graph over [rows][cols] float arrays, [cols] row vectors (broadcast down the
 * rows), [rows] column vectors produced by row reductions, and scalars.  `grad` appends the
 * reverse-mode derivative sub-graph; `compile` fuses every maximal group of elementwise nodes
 * into one map kernel (several results of one group leave the same kernel), selects a
 * hand-written specialised kernel where the whole group matches one, and plans the reductions
 * between them; `launch` enqueues the planned kernels on a stream. */
enum vrhi_graph_reduce {
  VRHI_R_ROW_SUM = 0, VRHI_R_ROW_MAX = 1, VRHI_R_COL_SUM = 2, VRHI_R_SUM_ALL = 3, VRHI_R_MEAN_ALL = 4
};
VRHI_API int vrhi_graph_create(vrhi_device dev, uint64_t rows, uint64_t cols, vrhi_graph *out_graph);
VRHI_API int vrhi_graph_destroy(vrhi_graph g); /* NULL is accepted */
/* flags: bit 0 = never select a specialised kernel (every fused group runs the generic tape
 * kernel).  The environment variable VRHI_GRAPH_NO_SPECIALIZE=1 sets bit 0 at creation. */
VRHI_API int vrhi_graph_set_flags(vrhi_graph g, uint32_t flags);
/* shape: 0 = full [rows][cols]; 1 = row vector [cols]; 2 = column vector [rows]; 3 = scalar. */
enum { VRHI_SHAPE_FULL = 0, VRHI_SHAPE_ROWVEC = 1, VRHI_SHAPE_COLVEC = 2, VRHI_SHAPE_SCALAR = 3 };
VRHI_API int vrhi_graph_input(vrhi_graph g, vrhi_buffer buf, int shape, int *out_node);
VRHI_API int vrhi_graph_const(vrhi_graph g, float value, int *out_node);
VRHI_API int vrhi_graph_unary(vrhi_graph g, int tape_op, int a, int *out_node);
VRHI_API int vrhi_graph_binary(vrhi_graph g, int tape_op, int a, int b, int *out_node);
VRHI_API int vrhi_graph_reduce(vrhi_graph g, int reduce_op, int a, int *out_node);
VRHI_API int vrhi_graph_softmax(vrhi_graph g, int a, int *out_node);
/* Append d(loss)/d(wrt[k]) for each k; loss must be a scalar node.  out_nodes[k] has the shape
 * of wrt[k] (a row-vector input receives a column reduction of its broadcast gradient). */
VRHI_API int vrhi_graph_grad(vrhi_graph g, int loss_node, const int *wrt, int n_wrt, int *out_nodes);
/* Mark `node` as a result to be written to `buf` (must hold the node's shape in floats). */
VRHI_API int vrhi_graph_output(vrhi_graph g, int node, vrhi_buffer buf);
VRHI_API int vrhi_graph_compile(vrhi_graph g);
VRHI_API int vrhi_graph_launch(vrhi_graph g, vrhi_stream stream);
/* Text plan of the compiled graph (one line per kernel); returns the needed length. */
VRHI_API int vrhi_graph_describe(vrhi_graph g, char *out_text, size_t capacity, size_t *out_needed);
VRHI_API int vrhi_graph_kernel_count(vrhi_graph g, int *out_count);

#ifdef __cplusplus
}
#endif
#endif /* VRHI_H_ */
