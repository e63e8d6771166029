"""ctypes binding of ``libvrhi.so`` (declared in ``include/vrhi.h``).

The shared object is built in-tree by ``vernondsl_b200/csrc/Makefile``.  There is no fallback:
if it is missing the import of anything that needs it raises, and every non-zero status from the
library becomes a :class:`VrhiError` carrying ``vrhi_last_error()``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvrhi.so")
CSRC = os.path.join(_HERE, "csrc")

# status codes (include/vrhi.h: enum vrhi_status)
OK, ERR_INVALID, ERR_CUDA, ERR_OOM, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_NOT_FOUND, ERR_SIZE, ERR_GRAPH, ERR_PEER = (
    0, -1, -2, -3, -4, -5, -6, -7, -8, -9)
STATUS_NAMES = {0: "VRHI_OK", -1: "VRHI_ERR_INVALID", -2: "VRHI_ERR_CUDA", -3: "VRHI_ERR_OOM",
                -4: "VRHI_ERR_UNSUPPORTED", -5: "VRHI_ERR_TIMEOUT", -6: "VRHI_ERR_NOT_FOUND",
                -7: "VRHI_ERR_SIZE", -8: "VRHI_ERR_GRAPH", -9: "VRHI_ERR_PEER"}

# argument classes: the vernon.semantic vocabulary (VernonToSpirv.cpp:44-55, color.mlir:9,44)
INPUT, OUTPUT, UNIFORM, UNIFORM_CONSTANT, STORAGE_BUFFER, IMAGE, VARYING = range(7)

MANDELBROT, JULIA = 0, 1
EXACT, FAST = 0, 1
ESCAPE_FLAG_CHECKED_ONLY = 1
TEST_NORM2_GT, TEST_NORM_GE = 0, 1
OUT_COUNT_U32, OUT_COUNT_U16, OUT_COLOR_F32 = 0, 1, 2
PART_CONTIGUOUS, PART_CYCLIC = 0, 1

TAPE_OPS = ["const", "add", "sub", "mul", "div", "max", "min", "fma", "neg", "abs", "square", "sqrt",
            "rsqrt", "recip", "exp", "log", "tanh", "sigmoid", "relu", "cos", "sin", "sign", "step", "eq"]
T = {name: k for k, name in enumerate(TAPE_OPS)}
TAPE_MAX_INSTR, TAPE_MAX_INPUTS, TAPE_MAX_OUTPUTS = 64, 8, 4
R_ROW_SUM, R_ROW_MAX, R_COL_SUM, R_SUM_ALL, R_MEAN_ALL = range(5)
SHAPE_FULL, SHAPE_ROWVEC, SHAPE_COLVEC, SHAPE_SCALAR = range(4)


class VrhiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


class DeviceProps(C.Structure):
    _fields_ = [("size", C.c_uint32), ("ordinal", C.c_int32), ("sm_count", C.c_int32),
                ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("sm_clock_khz", C.c_int32),
                ("mem_clock_khz", C.c_int32), ("l2_bytes", C.c_int32),
                ("smem_per_block_optin", C.c_int32), ("total_mem_bytes", C.c_uint64),
                ("name", C.c_char * 128)]


class Arg(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("offset", C.c_uint64), ("bytes", C.c_uint64),
                ("arg_class", C.c_int32), ("reserved", C.c_int32)]


class EscapeParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("kind", C.c_uint32), ("mode", C.c_uint32), ("test", C.c_uint32),
                ("output", C.c_uint32), ("width", C.c_uint32), ("height", C.c_uint32),
                ("max_iter", C.c_uint32), ("x0", C.c_float), ("y0", C.c_float), ("dx", C.c_float),
                ("dy", C.c_float), ("cr", C.c_float), ("ci", C.c_float), ("bound", C.c_float),
                ("color_scale", C.c_float), ("chunk_rows", C.c_uint32), ("chunk_first", C.c_uint32),
                ("chunk_step", C.c_uint32), ("chunk_count", C.c_uint32), ("flags", C.c_uint32)]


class WidenParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("width", C.c_uint32), ("height", C.c_uint32), ("chunk_rows", C.c_uint32),
                ("world", C.c_uint32), ("skip_rank", C.c_uint32), ("slab_first", C.c_uint32), ("slab_count", C.c_uint32),
                ("slab_stride", C.c_uint32)]


class GatherParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("width", C.c_uint32), ("height", C.c_uint32), ("chunk_rows", C.c_uint32),
                ("world", C.c_uint32), ("rank", C.c_uint32), ("slab_first", C.c_uint32), ("slab_count", C.c_uint32),
                ("seq", C.c_uint32), ("wait_ms", C.c_uint32), ("slab_stride", C.c_uint32)]


GATHER_MAX_WORLD = 8


class MapParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("reserved", C.c_uint32), ("n", C.c_uint64)]


class TapeInstr(C.Structure):
    _fields_ = [("op", C.c_uint16), ("a", C.c_uint16), ("b", C.c_uint16), ("c", C.c_uint16),
                ("imm", C.c_float)]


class TapeParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("n_inputs", C.c_uint32), ("n_outputs", C.c_uint32),
                ("n_instr", C.c_uint32), ("rows", C.c_uint64), ("cols", C.c_uint64),
                ("row_vector_mask", C.c_uint32), ("col_vector_mask", C.c_uint32),
                ("scalar_mask", C.c_uint32), ("out_value", C.c_uint32 * TAPE_MAX_OUTPUTS),
                ("instr", TapeInstr * TAPE_MAX_INSTR), ("flags", C.c_uint32), ("colsum_mask", C.c_uint32)]


TAPE_FLAG_INTERPRET = 1


class RowsParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("reserved", C.c_uint32), ("rows", C.c_uint64), ("cols", C.c_uint64)]


class MseParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("reserved", C.c_uint32), ("rows", C.c_uint64), ("cols", C.c_uint64),
                ("denom", C.c_double)]


class ProbeParams(C.Structure):
    _fields_ = [("size", C.c_uint32), ("variant", C.c_uint32), ("ffma_per_thread", C.c_uint64),
                ("threads", C.c_uint64)]


class RowPartition(C.Structure):
    _fields_ = [("chunk_rows", C.c_uint32), ("chunk_first", C.c_uint32), ("chunk_step", C.c_uint32),
                ("chunk_count", C.c_uint32), ("rows_owned", C.c_uint64)]


_vp, _i, _u64, _sz = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t
_P = C.POINTER
_u32 = C.c_uint32
# int (*vrhi_allgather_fn)(void *user, const void *send, void *recv, uint64_t bytes)
ALLGATHER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64)

# name -> argtypes; every function returns int unless listed in _RESTYPES
PROTOTYPES = {
    "vrhi_last_error": [],
    "vrhi_version": [],
    "vrhi_arg_class_from_semantic": [C.c_char_p, _P(_i)],
    "vrhi_arg_class_name": [_i],
    "vrhi_device_count": [_P(_i)],
    "vrhi_device_create": [_i, _P(_vp)],
    "vrhi_device_destroy": [_vp],
    "vrhi_device_props_get": [_vp, _P(DeviceProps)],
    "vrhi_device_synchronize": [_vp],
    "vrhi_device_set_alloc_limit": [_vp, _u64],
    "vrhi_device_allocated": [_vp, _P(_u64)],
    "vrhi_buffer_create": [_vp, _u64, _i, _P(_vp)],
    "vrhi_buffer_wrap": [_vp, _vp, _u64, _i, _P(_vp)],
    "vrhi_buffer_destroy": [_vp],
    "vrhi_buffer_size": [_vp, _P(_u64)],
    "vrhi_buffer_class": [_vp, _P(_i)],
    "vrhi_buffer_device_ptr": [_vp, _P(_vp)],
    "vrhi_buffer_upload": [_vp, _u64, _vp, _u64, _vp],
    "vrhi_buffer_download": [_vp, _u64, _vp, _u64, _vp],
    "vrhi_buffer_fill_u8": [_vp, _u64, _i, _u64, _vp],
    "vrhi_host_alloc": [_u64, _P(_vp)],
    "vrhi_host_free": [_vp],
    "vrhi_buffer_copy_2d": [_vp, _u64, _u64, _vp, _u64, _u64, _u64, _u64, _vp],
    "vrhi_buffer_ipc_export": [_vp, _vp],
    "vrhi_buffer_ipc_open": [_vp, _vp, _u64, _i, _P(_vp)],
    "vrhi_stream_create": [_vp, _P(_vp)],
    "vrhi_stream_wrap": [_vp, _vp, _P(_vp)],
    "vrhi_stream_destroy": [_vp],
    "vrhi_stream_synchronize": [_vp],
    "vrhi_stream_check": [_vp],
    "vrhi_stream_launch_count": [_vp, _P(_u64)],
    "vrhi_event_create": [_vp, _P(_vp)],
    "vrhi_event_destroy": [_vp],
    "vrhi_event_record": [_vp, _vp],
    "vrhi_event_synchronize": [_vp],
    "vrhi_event_elapsed_ms": [_vp, _vp, _P(C.c_float)],
    "vrhi_stream_wait_event": [_vp, _vp],
    "vrhi_tape_jit_stats": [_P(C.c_uint64), _P(C.c_uint64), _P(C.c_int), _P(C.c_int)],
    "vrhi_tape_source": [_P(TapeParams), C.c_char_p, C.c_uint64, _P(C.c_uint64)],
    "vrhi_sequence_begin": [_vp],
    "vrhi_sequence_fork": [_vp, _vp],
    "vrhi_sequence_end": [_vp, _P(_vp)],
    "vrhi_sequence_launch": [_vp, _vp],
    "vrhi_sequence_stats": [_vp, _P(C.c_uint64), _P(C.c_uint64), _P(C.c_uint64)],
    "vrhi_sequence_destroy": [_vp],
    "vrhi_op_count": [_P(_i)],
    "vrhi_op_name": [_i, _P(C.c_char_p)],
    "vrhi_op_lookup": [C.c_char_p, _P(_i)],
    "vrhi_op_signature": [_i, _P(C.c_char_p)],
    "vrhi_op_launch": [_vp, _i, _P(Arg), _i, _vp, _sz],
    "vrhi_col_sum_static_scratch": [_vp, _vp, _u64, _u64, _vp],
    "vrhi_partition_rows": [_u64, C.c_uint32, C.c_uint32, C.c_uint32, _i, _P(RowPartition)],
    "vrhi_partition_leading": [_u64, C.c_uint32, C.c_uint32, _P(_u64), _P(_u64)],
    "vrhi_group_create": [_vp, _u32, _u32, ALLGATHER_FN, _vp, _P(_vp)],
    "vrhi_group_destroy": [_vp],
    "vrhi_group_info": [_vp, _P(_u32), _P(_u32)],
    "vrhi_group_set_wait_ms": [_vp, _u32],
    "vrhi_group_all_reduce_sum_f32": [_vp, _vp, _u64, _u64, _vp],
    "vrhi_exchange_create": [_vp, _vp, _u32, _u32, _u32, _P(_vp)],
    "vrhi_exchange_destroy": [_vp],
    "vrhi_exchange_planes": [_vp, _P(_vp), _P(_vp)],
    "vrhi_exchange_publish": [_vp, _vp, _u32, _u32, _u32],
    "vrhi_exchange_complete": [_vp, _vp],
    "vrhi_exchange_check": [_vp],
    "vrhi_exchange_launch_count": [_vp, _P(_u64)],
    "vrhi_graph_create": [_vp, _u64, _u64, _P(_vp)],
    "vrhi_graph_destroy": [_vp],
    "vrhi_graph_set_flags": [_vp, C.c_uint32],
    "vrhi_graph_input": [_vp, _vp, _i, _P(_i)],
    "vrhi_graph_const": [_vp, C.c_float, _P(_i)],
    "vrhi_graph_unary": [_vp, _i, _i, _P(_i)],
    "vrhi_graph_binary": [_vp, _i, _i, _i, _P(_i)],
    "vrhi_graph_reduce": [_vp, _i, _i, _P(_i)],
    "vrhi_graph_softmax": [_vp, _i, _P(_i)],
    "vrhi_graph_grad": [_vp, _i, _P(_i), _i, _P(_i)],
    "vrhi_graph_output": [_vp, _i, _vp],
    "vrhi_graph_compile": [_vp],
    "vrhi_graph_launch": [_vp, _vp],
    "vrhi_graph_describe": [_vp, C.c_char_p, _sz, _P(_sz)],
    "vrhi_graph_kernel_count": [_vp, _P(_i)],
}
_RESTYPES = {"vrhi_last_error": C.c_char_p, "vrhi_arg_class_name": C.c_char_p}


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile libvrhi.so for sm_100a with nvcc (no GPU needed)."""
    cmd = ["make", "-C", CSRC, "-j", str(min(16, os.cpu_count() or 4))]
    if force:
        cmd.append("-B")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode:
        print(proc.stdout)
    if proc.returncode:
        raise RuntimeError("building libvrhi.so failed (see output above)")
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C {CSRC}` "
                "(or vernondsl_b200.build()); this package has no fallback implementation")
        L = C.CDLL(LIB_PATH)
        for name, argtypes in PROTOTYPES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export it
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        msg = lib().vrhi_last_error()
        raise VrhiError(status, msg.decode() if msg else "")
