// Run-time compilation of fused elementwise tapes.
//
// The interpreter in k_map.cu runs any tape but pays for decoding and for keeping every value in
// shared memory: a chain of a dozen operations is bound by instruction issue at well under half
// of the HBM roofline.  Here the same SSA tape is written out as the body of a CUDA kernel,
// compiled for sm_100a with NVRTC, loaded through the driver API and cached by its text; values
// live in registers and the kernel is bound by HBM like the hand-written chain kernel.
//
// Same arithmetic as the interpreter, operation by operation: additions, subtractions and
// multiplications are emitted as __fadd_rn / __fsub_rn / __fmul_rn so that the compiler cannot
// contract two tape operations into one fused multiply-add, fused multiply-adds appear only where
// the tape says so, and the transcendental primitives are the same functions (tape_math.cuh is
// compiled into both).  The two paths therefore produce the same bits.
//
// NVRTC and the driver entry points are looked up at run time (dlopen, cudaGetDriverEntryPoint):
// the library neither links against them nor needs them unless a tape is launched.  Where NVRTC is
// not installed the interpreter runs instead; VRHI_TAPE_JIT=0 in the environment, or
// VRHI_TAPE_FLAG_INTERPRET in the parameter block, selects the interpreter explicitly.
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "vrhi_internal.h"

namespace vrhi {

namespace {

const char kMathSource[] =
#include "tape_math_src.inc"
    ;

struct Nvrtc {
  decltype(&nvrtcCreateProgram) create = nullptr;
  decltype(&nvrtcCompileProgram) compile = nullptr;
  decltype(&nvrtcGetCUBINSize) cubin_size = nullptr;
  decltype(&nvrtcGetCUBIN) cubin = nullptr;
  decltype(&nvrtcGetProgramLogSize) log_size = nullptr;
  decltype(&nvrtcGetProgramLog) log = nullptr;
  decltype(&nvrtcDestroyProgram) destroy = nullptr;
  decltype(&nvrtcGetErrorString) error_string = nullptr;
  decltype(&nvrtcVersion) version = nullptr;
  int version_number = 0;  // major * 1000 + minor * 10, as CUDART_VERSION counts
  bool ok = false;
};

struct Driver {
  CUresult (*module_load_data)(CUmodule *, const void *) = nullptr;
  CUresult (*module_get_function)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*launch_kernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void **,
                            void **) = nullptr;
  CUresult (*get_error_string)(CUresult, const char **) = nullptr;
  CUresult (*occupancy)(int *, CUfunction, int, size_t) = nullptr;
  bool ok = false;
};

std::mutex g_mu;
Nvrtc g_nvrtc;
Driver g_driver;
bool g_loaded = false;
uint64_t g_compiled = 0, g_launches = 0;
struct Compiled {
  CUfunction fn;
  bool flat;     // no row or column vectors: the kernel indexes the data as one long array
  int resident;  // blocks of 256 threads that fit on one SM at a time
};
std::unordered_map<std::string, Compiled> g_cache;  // key: device ordinal + the tape's description

template <class F>
bool sym(void *lib, const char *name, F *out) {
  *out = reinterpret_cast<F>(dlsym(lib, name));
  return *out != nullptr;
}

template <class F>
bool drv(const char *name, F *out) {
  void *p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    (void)cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(p);
  return true;
}

bool bind(void *lib, Nvrtc *out) {
  Nvrtc n;
  n.ok = sym(lib, "nvrtcCreateProgram", &n.create) && sym(lib, "nvrtcCompileProgram", &n.compile) &&
         sym(lib, "nvrtcGetCUBINSize", &n.cubin_size) && sym(lib, "nvrtcGetCUBIN", &n.cubin) &&
         sym(lib, "nvrtcGetProgramLogSize", &n.log_size) && sym(lib, "nvrtcGetProgramLog", &n.log) &&
         sym(lib, "nvrtcDestroyProgram", &n.destroy) && sym(lib, "nvrtcGetErrorString", &n.error_string) &&
         sym(lib, "nvrtcVersion", &n.version);
  if (!n.ok) return false;
  int major = 0, minor = 0;
  if (n.version(&major, &minor) != NVRTC_SUCCESS) return false;
  n.version_number = major * 1000 + minor * 10;
  *out = n;
  return true;
}

void load_once() {
  if (g_loaded) return;
  g_loaded = true;
  // The compiler whose version is the one this library was built with is preferred: its math
  // library is then the one the interpreting kernel was compiled against, which is what makes the
  // two paths agree bit for bit.  Any other NVRTC 12 still gives a correct kernel.
  const char *names[] = {getenv("VRHI_NVRTC"), "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.12", "libnvrtc.so"};
  Nvrtc fallback;
  for (const char *name : names) {
    if (!name || !*name) continue;
    void *lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    Nvrtc n;
    if (!lib || !bind(lib, &n)) continue;
    if (n.version_number / 10 == CUDART_VERSION / 10) { g_nvrtc = n; break; }
    if (!fallback.ok) fallback = n;
  }
  if (!g_nvrtc.ok && fallback.ok) g_nvrtc = fallback;
  Driver &d = g_driver;
  d.ok = drv("cuModuleLoadData", &d.module_load_data) && drv("cuModuleGetFunction", &d.module_get_function) &&
         drv("cuLaunchKernel", &d.launch_kernel) && drv("cuGetErrorString", &d.get_error_string) &&
         drv("cuOccupancyMaxActiveBlocksPerMultiprocessor", &d.occupancy);
}

std::string v(unsigned k) { return "v" + std::to_string(k); }

// One SSA instruction as a C expression over the values v<k>.
std::string expression(const vrhi_tape_instr &I) {
  const std::string a = v(I.a), b = v(I.b), c = v(I.c);
  switch (I.op) {
    case VRHI_T_CONST: {
      uint32_t bits;
      memcpy(&bits, &I.imm, 4);
      char buf[48];
      snprintf(buf, sizeof buf, "__int_as_float((int)0x%08xu)", bits);
      return buf;
    }
    case VRHI_T_ADD: return "__fadd_rn(" + a + ", " + b + ")";
    case VRHI_T_SUB: return "__fsub_rn(" + a + ", " + b + ")";
    case VRHI_T_MUL: return "__fmul_rn(" + a + ", " + b + ")";
    case VRHI_T_DIV: return a + " / " + b;
    case VRHI_T_MAX: return "fmaxf(" + a + ", " + b + ")";
    case VRHI_T_MIN: return "fminf(" + a + ", " + b + ")";
    case VRHI_T_EQ: return "(" + a + " == " + b + " ? 1.f : 0.f)";
    case VRHI_T_FMA: return "fmaf(" + a + ", " + b + ", " + c + ")";
    case VRHI_T_NEG: return "-" + a;
    case VRHI_T_ABS: return "fabsf(" + a + ")";
    case VRHI_T_SQUARE: return "__fmul_rn(" + a + ", " + a + ")";
    case VRHI_T_RELU: return "fmaxf(" + a + ", 0.0f)";
    case VRHI_T_SIGN: return "((" + a + " > 0.f) ? 1.f : ((" + a + " < 0.f) ? -1.f : 0.f))";
    case VRHI_T_STEP: return "(" + a + " > 0.f ? 1.f : 0.f)";
    case VRHI_T_SQRT: return "sqrtf(" + a + ")";
    case VRHI_T_RSQRT: return "1.0f / sqrtf(" + a + ")";
    case VRHI_T_RECIP: return "1.0f / " + a;
    case VRHI_T_EXP: return "expf(" + a + ")";
    case VRHI_T_LOG: return "logf(" + a + ")";
    case VRHI_T_TANH: return "tanhf(" + a + ")";
    case VRHI_T_SIGMOID: return "sigmoid_accurate(" + a + ")";
    case VRHI_T_COS: return "cosf(" + a + ")";
    default: return "sinf(" + a + ")";  // VRHI_T_SIN
  }
}

// The kernel: 256 threads, each owning one float4 column group; blockIdx.y strides over rows, `unroll`
// rows per trip with the loads of all of them issued before any is used.  Row vectors are
// loaded once per thread, column vectors once per row, scalars once per thread.  Without row or
// column vectors the data is one long array (`flat`): the host picks a convenient row length.
std::string generate(const vrhi_tape_params &q, bool *flat_out, int unroll = 2) {
  const unsigned NI = q.n_inputs, NO = q.n_outputs, NT = q.n_instr;
  const bool flat = (q.row_vector_mask | q.col_vector_mask) == 0 && q.colsum_mask == 0;  // column sums need a thread to keep its columns
  *flat_out = flat;
  std::vector<bool> used(NI + NT, false);
  for (unsigned t = 0; t < NT; ++t) {
    const int ar = tape_arity(q.instr[t].op);
    const uint16_t src[3] = {q.instr[t].a, q.instr[t].b, q.instr[t].c};
    for (int s = 0; s < ar; ++s) used[src[s]] = true;
  }
  for (unsigned k = 0; k < NO; ++k) used[q.out_value[k]] = true;
  auto shape = [&](unsigned k) { return ((q.row_vector_mask >> k) & 1u) ? 'r' : ((q.col_vector_mask >> k) & 1u) ? 'c' : ((q.scalar_mask >> k) & 1u) ? 's' : 'f'; };

  std::string s = kMathSource;
  s += "\n__device__ __forceinline__ void tape_body(";
  for (unsigned k = 0; k < NI; ++k) s += "const float " + v(k) + ", ";
  for (unsigned k = 0; k < NO; ++k) s += "float &r" + std::to_string(k) + (k + 1 < NO ? ", " : "");
  s += ") {\n";
  for (unsigned t = 0; t < NT; ++t) s += "  const float " + v(NI + t) + " = " + expression(q.instr[t]) + ";\n";
  for (unsigned k = 0; k < NO; ++k) s += "  r" + std::to_string(k) + " = " + v(q.out_value[k]) + ";\n";
  s += "}\n\nextern \"C\" __global__ void __launch_bounds__(256) vrhi_tape_kernel(";
  for (unsigned k = 0; k < NI; ++k) s += "const float *__restrict__ in" + std::to_string(k) + ", ";
  for (unsigned k = 0; k < NO; ++k) s += "float *__restrict__ out" + std::to_string(k) + ", ";
  s += "const unsigned long long n4, const unsigned long long rows, const unsigned long long rows_full, const unsigned int cols4) {\n";
  s += "  const unsigned int c4 = blockIdx.x * 256u + threadIdx.x;\n  if (c4 >= cols4) return;\n";
  for (unsigned k = 0; k < NI; ++k) {
    if (!used[k]) continue;
    const std::string K = std::to_string(k);
    if (shape(k) == 'r') s += "  const float4 x" + K + " = __ldg(reinterpret_cast<const float4 *>(in" + K + ") + c4);\n";
    if (shape(k) == 's') s += "  const float s" + K + " = __ldg(in" + K + ");\n  const float4 x" + K + " = make_float4(s" + K + ", s" + K + ", s" + K + ", s" + K + ");\n";
  }
  // loads of one row group, and its arithmetic and stores
  auto loads = [&](const std::string &G, const std::string &idx, const std::string &row) {
    std::string t;
    for (unsigned k = 0; k < NI; ++k) {
      if (!used[k]) continue;
      const std::string K = std::to_string(k), name = "x" + K + "_" + G;
      if (shape(k) == 'f') t += "      const float4 " + name + " = __ldcs(reinterpret_cast<const float4 *>(in" + K + ") + " + idx + ");\n";
      if (shape(k) == 'c') t += "      const float c" + K + "_" + G + " = __ldg(in" + K + " + " + row + ");\n      const float4 " + name + " = make_float4(c" + K + "_" + G + ", c" + K + "_" + G + ", c" + K + "_" + G + ", c" + K + "_" + G + ");\n";
    }
    return t;
  };
  auto work = [&](const std::string &G, const std::string &idx) {
    std::string t = "      {\n";
    for (unsigned k = 0; k < NO; ++k) t += "        float4 o" + std::to_string(k) + ";\n";
    for (const char *comp : {"x", "y", "z", "w"}) {
      t += "        tape_body(";
      for (unsigned k = 0; k < NI; ++k) {
        const std::string K = std::to_string(k);
        if (!used[k]) t += "0.0f, ";
        else if (shape(k) == 'r' || shape(k) == 's') t += "x" + K + "." + comp + ", ";
        else t += "x" + K + "_" + G + "." + comp + ", ";
      }
      for (unsigned k = 0; k < NO; ++k) t += "o" + std::to_string(k) + "." + comp + (k + 1 < NO ? ", " : "");
      t += ");\n";
    }
    for (unsigned k = 0; k < NO; ++k) {
      const std::string K = std::to_string(k);
      if ((q.colsum_mask >> k) & 1u)  // rows are visited in a fixed order: the sum does not depend on scheduling
        t += "        acc" + K + ".x += o" + K + ".x; acc" + K + ".y += o" + K + ".y; acc" + K + ".z += o" + K + ".z; acc" + K + ".w += o" + K + ".w;\n";
      else
        t += "        __stcs(reinterpret_cast<float4 *>(out" + K + ") + " + idx + ", o" + K + ");\n";
    }
    return t + "      }\n";
  };
  for (unsigned k = 0; k < NO; ++k)
    if ((q.colsum_mask >> k) & 1u) s += "  float4 acc" + std::to_string(k) + " = make_float4(0.f, 0.f, 0.f, 0.f);\n";
  s += "  unsigned long long row = blockIdx.y;\n";
  const std::string U = std::to_string(unroll);
  s += "  for (; row + " + std::to_string(unroll - 1) + "ull * gridDim.y < rows_full; row += " + U + "ull * gridDim.y) {  // " + U + " complete rows per trip: all loads first\n";
  for (int g = 0; g < unroll; ++g) {
    const std::string G = std::to_string(g);
    s += "      const unsigned long long row_" + G + " = row + " + G + "ull * gridDim.y, i" + G + " = row_" + G + " * cols4 + c4;\n";
  }
  for (int g = 0; g < unroll; ++g) s += loads(std::to_string(g), "i" + std::to_string(g), "row_" + std::to_string(g));
  for (int g = 0; g < unroll; ++g) s += work(std::to_string(g), "i" + std::to_string(g));
  s += "  }\n";
  s += "  for (; row < rows; row += gridDim.y) {  // rows left over; the last one may be ragged\n";
  s += "      const unsigned long long i0 = row * cols4 + c4;\n      if (i0 >= n4) break;\n";
  s += loads("0", "i0", "row") + work("0", "i0");
  s += "  }\n";
  // column-summed outputs: this block's partial row, [gridDim.y][cols]; a second kernel adds the partial rows
  for (unsigned k = 0; k < NO; ++k)
    if ((q.colsum_mask >> k) & 1u)
      s += "  reinterpret_cast<float4 *>(out" + std::to_string(k) + ")[(unsigned long long)blockIdx.y * cols4 + c4] = acc" + std::to_string(k) + ";\n";
  s += "}\n";
  return s;
}

int compile(vrhi_device_t *dev, const std::string &src, CUfunction *out) {
  nvrtcProgram prog = nullptr;
  nvrtcResult r = g_nvrtc.create(&prog, src.c_str(), "vrhi_tape.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) return fail(VRHI_ERR_CUDA, "nvrtcCreateProgram: %s", g_nvrtc.error_string(r));
  char arch[64];
  snprintf(arch, sizeof arch, "--gpu-architecture=sm_%d%d%s", dev->prop.major, dev->prop.minor, dev->prop.major >= 9 ? "a" : "");
  const char *opts[] = {arch, "--std=c++17", "-lineinfo"};
  r = g_nvrtc.compile(prog, 3, opts);
  if (r != NVRTC_SUCCESS) {
    size_t n = 0;
    g_nvrtc.log_size(prog, &n);
    std::string log(n ? n : 1, '\0');
    if (n) g_nvrtc.log(prog, &log[0]);
    g_nvrtc.destroy(&prog);
    return fail(VRHI_ERR_CUDA, "compiling a fused tape failed: %s\n%.1500s", g_nvrtc.error_string(r), log.c_str());
  }
  size_t bytes = 0;
  g_nvrtc.cubin_size(prog, &bytes);
  std::vector<char> image(bytes);
  r = g_nvrtc.cubin(prog, image.data());
  g_nvrtc.destroy(&prog);
  if (r != NVRTC_SUCCESS || bytes == 0) return fail(VRHI_ERR_CUDA, "nvrtcGetCUBIN: %s", g_nvrtc.error_string(r));
  CUmodule mod = nullptr;
  CUresult cr = g_driver.module_load_data(&mod, image.data());
  const char *msg = "?";
  if (cr != CUDA_SUCCESS) {
    g_driver.get_error_string(cr, &msg);
    return fail(VRHI_ERR_CUDA, "cuModuleLoadData: %s", msg);
  }
  cr = g_driver.module_get_function(out, mod, "vrhi_tape_kernel");
  if (cr != CUDA_SUCCESS) {
    g_driver.get_error_string(cr, &msg);
    return fail(VRHI_ERR_CUDA, "cuModuleGetFunction: %s", msg);
  }
  return VRHI_OK;  // the module stays loaded for the life of the process (it is in the cache)
}

}  // namespace

// Returns VRHI_OK when the compiled kernel was launched, 1 when this tape or shape is left to the
// interpreter (no NVRTC, switched off, columns not a multiple of 4, unaligned pointers), and an
// error code when compilation or the launch failed.
// VRHI_TAPE_JIT=0 in the environment selects the interpreting kernel for every tape; read once per process
static bool jit_enabled() {
  static const bool on = env_int("VRHI_TAPE_JIT", 0, 1, 1) != 0;
  return on;
}

int tape_jit_launch(vrhi_stream_t *st, const vrhi_tape_params &q, const float *const *in, float *const *out) {
  if (q.flags & VRHI_TAPE_FLAG_INTERPRET) return 1;
  if (!jit_enabled()) return 1;
  if (q.cols % 4 != 0) return 1;
  for (uint32_t k = 0; k < q.n_inputs; ++k)
    if (!((q.col_vector_mask >> k) & 1u) && !((q.scalar_mask >> k) & 1u) && ((uintptr_t)in[k] % 16)) return 1;
  for (uint32_t k = 0; k < q.n_outputs; ++k)
    if ((uintptr_t)out[k] % 16) return 1;

  std::lock_guard<std::mutex> lock(g_mu);
  load_once();
  if (!g_nvrtc.ok || !g_driver.ok) return 1;
  bool flat = false;
  // About three 16-byte loads in flight per thread and six blocks per SM, all resident at once (one wave):
  // measured on B200 with the three-input chain, 6.8 TB/s; eight blocks per SM spill into a second, partly
  // filled wave and two rows per trip then cost 15 %.
  int full_inputs = 0;
  for (uint32_t k = 0; k < q.n_inputs; ++k)
    if (!(((q.row_vector_mask | q.col_vector_mask | q.scalar_mask) >> k) & 1u)) ++full_inputs;
  int unroll = full_inputs >= 3 ? 1 : full_inputs == 2 ? 2 : 3, blocks_per_sm = 0;  // 0: what is resident at once, at most 6
  static const int env_unroll = env_int("VRHI_TAPE_UNROLL", 1, 8, 0), env_blocks = env_int("VRHI_TAPE_BLOCKS_PER_SM", 1, 32, 0);  // tuning aids
  if (env_unroll) unroll = env_unroll;
  if (env_blocks) blocks_per_sm = env_blocks;
  // cache key: everything the generated text depends on, as raw bytes (the text itself is only built on a miss)
  std::string key;
  {
    const uint32_t head[8] = {(uint32_t)st->dev->ordinal, (uint32_t)unroll, q.n_inputs, q.n_outputs, q.n_instr,
                              q.row_vector_mask, q.col_vector_mask, q.scalar_mask};
    key.append(reinterpret_cast<const char *>(head), sizeof head);
    key.append(reinterpret_cast<const char *>(q.out_value), sizeof(uint32_t) * q.n_outputs);
    key.append(reinterpret_cast<const char *>(&q.colsum_mask), sizeof q.colsum_mask);
    for (uint32_t t = 0; t < q.n_instr; ++t) {  // field by field: padding bytes of the struct are not defined
      const vrhi_tape_instr &I = q.instr[t];
      const uint16_t f[4] = {I.op, I.a, I.b, I.c};
      key.append(reinterpret_cast<const char *>(f), sizeof f);
      key.append(reinterpret_cast<const char *>(&I.imm), sizeof I.imm);
    }
  }
  auto it = g_cache.find(key);
  if (it == g_cache.end()) {
    const std::string src = generate(q, &flat, unroll);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    VRHI_CUDA(cudaStreamIsCapturing(st->s, &cap));
    if (cap != cudaStreamCaptureStatusNone)
      return fail(VRHI_ERR_INVALID, "this tape has not been compiled yet; run the operator once on the stream before recording it");
    VRHI_CUDA(cudaFree(nullptr));  // makes the device's primary context current for the driver calls below
    CUfunction fn = nullptr;
    VRHI_TRY(compile(st->dev, src, &fn));
    int resident = 0;
    if (g_driver.occupancy(&resident, fn, 256, 0) != CUDA_SUCCESS || resident < 1) resident = 4;
    it = g_cache.emplace(key, Compiled{fn, flat, resident}).first;
    ++g_compiled;
  }
  const uint64_t n4 = q.rows * q.cols / 4;
  uint64_t rows = q.rows;
  uint32_t cols4 = (uint32_t)(q.cols / 4);
  if (q.cols / 4 > 0xffffffffull) return 1;
  flat = it->second.flat;
  if (flat) {  // one long array: rows of 1024 float4 groups, the last one ragged (guarded by n4)
    cols4 = n4 < 1024 ? (uint32_t)n4 : 1024u;
    rows = (n4 + cols4 - 1) / cols4;
  }
  const unsigned gx = (cols4 + 255u) / 256u;
  if (blocks_per_sm == 0) blocks_per_sm = it->second.resident < 6 ? it->second.resident : 6;
  const uint64_t target = (uint64_t)st->dev->prop.multiProcessorCount * blocks_per_sm;
  uint64_t gy = (target + gx - 1) / gx;
  const uint64_t row_pairs = (rows + unroll - 1) / unroll;
  if (gy > row_pairs) gy = row_pairs;
  if (gy > 65535) gy = 65535;
  if (gy == 0) gy = 1;
  void *args[VRHI_TAPE_MAX_INPUTS + VRHI_TAPE_MAX_OUTPUTS + 4];
  const float *in_copy[VRHI_TAPE_MAX_INPUTS];
  float *out_copy[VRHI_TAPE_MAX_OUTPUTS];
  int n = 0;
  for (uint32_t k = 0; k < q.n_inputs; ++k) { in_copy[k] = in[k]; args[n++] = &in_copy[k]; }
  char *scratch = nullptr;
  if (q.colsum_mask) {
    const size_t per_output = (size_t)gy * q.cols * sizeof(float);
    VRHI_TRY(stream_arena(st, per_output * VRHI_TAPE_MAX_OUTPUTS, nullptr, &scratch));
  }
  for (uint32_t k = 0; k < q.n_outputs; ++k) {
    out_copy[k] = ((q.colsum_mask >> k) & 1u) ? reinterpret_cast<float *>(scratch + (size_t)k * gy * q.cols * sizeof(float)) : out[k];
    args[n++] = &out_copy[k];
  }
  uint64_t n4_arg = n4, rows_arg = rows, rows_full = n4 / cols4;  // rows_full: rows that hold all cols4 groups
  args[n++] = &n4_arg; args[n++] = &rows_arg; args[n++] = &rows_full; args[n++] = &cols4;
  CUresult cr = g_driver.launch_kernel(it->second.fn, gx, (unsigned)gy, 1, 256, 1, 1, 0, reinterpret_cast<CUstream>(st->s), args, nullptr);
  if (cr != CUDA_SUCCESS) {
    const char *msg = "?";
    g_driver.get_error_string(cr, &msg);
    return fail(VRHI_ERR_CUDA, "launch of a compiled tape failed: %s", msg);
  }
  ++g_launches;
  for (uint32_t k = 0; k < q.n_outputs; ++k)
    if ((q.colsum_mask >> k) & 1u) VRHI_TRY(col_finalize(st, out_copy[k], out[k], (uint32_t)gy, q.cols, 1.0f));
  return VRHI_OK;
}

bool tape_jit_available() {
  if (!jit_enabled()) return false;
  std::lock_guard<std::mutex> lock(g_mu);
  load_once();
  return g_nvrtc.ok && g_driver.ok;
}

void tape_jit_counters(uint64_t *compiled, uint64_t *launches, int *compiler_version, int *built_version) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (compiled) *compiled = g_compiled;
  if (launches) *launches = g_launches;
  if (compiler_version) *compiler_version = g_nvrtc.ok ? g_nvrtc.version_number : 0;
  if (built_version) *built_version = CUDART_VERSION / 10 * 10;
}

// The generated source of a tape, for inspection and for tests that run without a GPU.
std::string tape_jit_source(const vrhi_tape_params &q) {
  bool flat = false;
  return generate(q, &flat);
}

}  // namespace vrhi
