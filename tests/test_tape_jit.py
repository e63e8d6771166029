"""CPU: the source the library generates for a fused tape must be valid CUDA for sm_100a.  NVRTC
compiles without a device, so the generator is checked here; that the compiled kernels compute
the same bits as the interpreting kernel is checked on the GPU (tests/test_map_gpu.py)."""
import ctypes as C

import pytest

from vernondsl_b200 import ops


def _nvrtc():
    for name in ("libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"):
        try:
            return C.CDLL(name)
        except OSError:
            continue
    return None


def _compile(src: str):
    lib = _nvrtc()
    if lib is None:
        pytest.skip("NVRTC is not installed")
    prog = C.c_void_p()
    assert lib.nvrtcCreateProgram(C.byref(prog), src.encode(), b"vrhi_tape.cu", 0, None, None) == 0
    opts = (C.c_char_p * 2)(b"--gpu-architecture=sm_100a", b"--std=c++17")
    rc = lib.nvrtcCompileProgram(prog, 2, opts)
    n = C.c_size_t()
    lib.nvrtcGetProgramLogSize(prog, C.byref(n))
    log = C.create_string_buffer(max(n.value, 1))
    lib.nvrtcGetProgramLog(prog, log)
    size = C.c_size_t()
    lib.nvrtcGetCUBINSize(prog, C.byref(size))
    lib.nvrtcDestroyProgram(C.byref(prog))
    return rc, log.value.decode(errors="replace"), size.value


def _chain():
    t = ops.Tape(3)
    a, x, y = t.input(0), t.input(1), t.input(2)
    e = t.op("exp", t.op("mul", t.op("mul", t.const(-0.5), x), x))
    q = t.op("sqrt", t.op("add", t.op("abs", y), t.const(1e-3)))
    t.output(t.op("fma", t.op("tanh", t.op("fma", a, x, y)), e, q))
    return t


def _every_op():
    t = ops.Tape(2)
    x, y = t.input(0), t.input(1)
    acc = t.op("add", x, y)
    for name in ("sub", "mul", "div", "max", "min", "eq"):
        acc = t.op("add", acc, t.op(name, x, y))
    for name in ("neg", "abs", "square", "relu", "sign", "step", "sqrt", "rsqrt", "recip", "exp", "log", "tanh", "sigmoid", "cos", "sin"):
        acc = t.op("add", acc, t.op(name, x))
    t.output(t.op("fma", acc, t.const(0.5), y))
    t.output(t.op("sigmoid", y))
    return t


def _broadcasts():
    t = ops.Tape(5, row_vectors=[1], col_vectors=[2], scalars=[3])     # input 4 is never read
    s = t.op("add", t.op("mul", t.input(0), t.input(1)), t.input(2))
    t.output(s)
    t.output(t.op("mul", t.op("max", s, t.const(0.0)), t.input(3)))
    t.output(t.input(0))                                                # an input handed straight to an output
    return t


def _column_sum():
    t = ops.Tape(3, row_vectors=[2])
    u = t.op("tanh", t.op("fma", t.input(0), t.input(1), t.input(2)))
    t.output(u)
    t.output(t.op("mul", u, t.input(0)), col_sum=True)               # summed over the rows inside the kernel
    return t


@pytest.mark.parametrize("make", [_chain, _every_op, _broadcasts, _column_sum])
def test_generated_source_compiles_for_sm_100a(make):
    src = ops.tape_source(make())
    assert 'extern "C" __global__' in src and "tape_body" in src
    rc, log, size = _compile(src)
    assert rc == 0, log
    assert size > 0


def test_generated_source_keeps_tape_operations_apart():
    """A multiply followed by an add must not become a fused multiply-add: the interpreting kernel
    rounds after each operation, and both paths have to give the same bits."""
    src = ops.tape_source(_chain())
    body = src[src.index("void tape_body"):src.index('extern "C"')]
    assert "__fmul_rn" in body and "__fadd_rn" in body
    assert " * " not in body and " + " not in body
    assert body.count("fmaf(") == 2            # exactly the two fused multiply-adds the tape asks for
    assert "0xbf000000" in body                # -0.5, bit for bit
