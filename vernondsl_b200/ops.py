"""Operator launches through ``vrhi_op_launch``: one Python function per registered kernel.

Each function takes :class:`~vernondsl_b200.rhi.Buffer` arguments that already live on the
device, fills the operator's parameter struct and enqueues the kernel on a stream.  Nothing here
computes: a missing library or an unsupported shape raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib as L
from ._lib import check, lib
from .rhi import Buffer, Stream

_op_ids: dict = {}


def op_id(name: str) -> int:
    if name not in _op_ids:
        v = C.c_int()
        check(lib().vrhi_op_lookup(name.encode(), C.byref(v)))
        _op_ids[name] = v.value
    return _op_ids[name]


def op_names() -> list:
    n = C.c_int()
    check(lib().vrhi_op_count(C.byref(n)))
    out = []
    for k in range(n.value):
        s = C.c_char_p()
        check(lib().vrhi_op_name(k, C.byref(s)))
        out.append(s.value.decode())
    return out


def launch(stream: Stream, name: str, args: Sequence[L.Arg], params) -> None:
    arr = (L.Arg * len(args))(*args)
    check(lib().vrhi_op_launch(stream._h, op_id(name), arr, len(args), C.byref(params), C.sizeof(params)))


# ------------------------------------------------------------------------------ escape time ---
def grid_steps(x0: float, x1: float, y0: float, y1: float, width: int, height: int):
    """Per-pixel steps in binary32: dx = (x1 - x0) / width, dy = (y1 - y0) / height.
    Index i maps to x0 + i*dx: the pixel corner, as fractal.py:20 maps i to (i/n - 1)*2."""
    f = np.float32
    return f((f(x1) - f(x0)) / f(width)), f((f(y1) - f(y0)) / f(height))


def escape_params(kind: int, width: int, height: int, x0: float, y0: float, dx: float, dy: float, *, cr: float = 0.0,
                  ci: float = 0.0, max_iter: int = 256, mode: int = L.EXACT, test: int = L.TEST_NORM2_GT,
                  bound: float = 4.0, output: int = L.OUT_COUNT_U32, color_scale: float = 0.0,
                  partition: Optional[L.RowPartition] = None, checked_only: bool = False,
                  transposed: bool = False, independent_of: int = 0) -> L.EscapeParams:
    """``independent_of`` = k (0..7): the launch touches nothing that the k escape_time launches before it on its
    stream write (a ring of k+1 frames), and may begin before they end."""
    if not 0 <= independent_of <= 7:
        raise ValueError("independent_of: 0..7")
    p = L.EscapeParams()
    p.size = C.sizeof(L.EscapeParams)
    p.kind, p.mode, p.test, p.output = kind, mode, test, output
    p.width, p.height, p.max_iter = width, height, max_iter
    p.x0, p.y0, p.dx, p.dy = x0, y0, dx, dy
    p.cr, p.ci, p.bound, p.color_scale = cr, ci, bound, color_scale
    p.flags = (1 if checked_only else 0) | (2 if transposed else 0) | (independent_of << 8)
    if partition is not None:
        p.chunk_rows, p.chunk_first = partition.chunk_rows, partition.chunk_first
        p.chunk_step, p.chunk_count = partition.chunk_step, partition.chunk_count
    return p


def escape_time(stream: Stream, image: Buffer, params: L.EscapeParams, wire: Optional[Buffer] = None,
                byte_plane: Optional[Buffer] = None) -> None:
    """Launch the escape-time map (the per-pixel loop of fractal.py:18-25) into ``image``.  ``wire``,
    a uint16 image of the same geometry, receives every count a second time (the form sent to peers);
    ``byte_plane`` (with ``wire``), a uint8 plane, receives min(count, 255)."""
    args = [image.arg(L.IMAGE if image.arg_class == L.IMAGE else L.OUTPUT)]
    if wire is not None:
        args.append(wire.arg(L.IMAGE if wire.arg_class == L.IMAGE else L.OUTPUT))
        if byte_plane is not None:
            args.append(byte_plane.arg(L.IMAGE if byte_plane.arg_class == L.IMAGE else L.OUTPUT))
    launch(stream, "escape_time", args, params)


def widen_rows_u16(stream: Stream, wire: Buffer, image: Buffer, width: int, height: int, chunk_rows: int, world: int,
                   skip_rank: int, slab_first: int, slab_count: int, slab_stride: int = 1) -> None:
    """Copy uint16 counts of slabs ``slab_first + k*slab_stride`` (k < slab_count) into the uint32 image, leaving out
    ``skip_rank``'s chunks."""
    p = L.WidenParams()
    p.size = C.sizeof(L.WidenParams)
    p.width, p.height, p.chunk_rows, p.world = int(width), int(height), int(chunk_rows), int(world)
    p.skip_rank, p.slab_first, p.slab_count, p.slab_stride = int(skip_rank), int(slab_first), int(slab_count), int(slab_stride)
    launch(stream, "widen_rows_u16", [wire.arg(), image.arg(L.IMAGE if image.arg_class == L.IMAGE else L.OUTPUT)], p)


def widen_rows_u8(stream: Stream, byte_plane: Buffer, image: Buffer, wires: Sequence[Buffer], width: int, height: int, chunk_rows: int,
                  world: int, skip_rank: int, slab_first: int, slab_count: int, slab_stride: int = 1) -> None:
    """Byte plane -> uint32 image for the given slabs; granules showing a byte of 255 come from ``wires[owner]``."""
    p = L.WidenParams()
    p.size = C.sizeof(L.WidenParams)
    p.width, p.height, p.chunk_rows, p.world, p.skip_rank = int(width), int(height), int(chunk_rows), int(world), int(skip_rank)
    p.slab_first, p.slab_count, p.slab_stride = int(slab_first), int(slab_count), int(slab_stride)
    launch(stream, "widen_rows_u8", [byte_plane.arg(L.INPUT), image.arg(L.IMAGE if image.arg_class == L.IMAGE else L.OUTPUT)] +
           [w.arg(L.INPUT) for w in wires], p)


def gather_signal(stream: Stream, peer_flags: Sequence[Buffer], world: int, rank: int, seq: int) -> None:
    """Store ``seq`` into slot ``rank`` of every peer's flag array: this rank's rows up to that number are ready."""
    p = L.GatherParams()
    p.size, p.world, p.rank, p.seq = C.sizeof(L.GatherParams), int(world), int(rank), int(seq) & 0xFFFFFFFF
    launch(stream, "gather_signal", [f.arg(L.STORAGE_BUFFER) for f in peer_flags], p)


def gather_pull_u16(stream: Stream, flags: Buffer, image: Buffer, peer_wires: Sequence[Buffer], width: int, height: int,
                    chunk_rows: int, world: int, rank: int, slab_first: int, slab_count: int, seq: int, wait_ms: int = 0,
                    slab_stride: int = 1) -> None:
    """Wait (bounded) for every peer's flag to reach ``seq``, then read the peers' uint16 rows of the given slabs out
    of their wire images and write them, widened, into ``image``.  ``peer_wires``: ranks in order, without ``rank``."""
    p = L.GatherParams()
    p.size = C.sizeof(L.GatherParams)
    p.width, p.height, p.chunk_rows, p.world, p.rank = int(width), int(height), int(chunk_rows), int(world), int(rank)
    p.slab_first, p.slab_count, p.seq, p.wait_ms = int(slab_first), int(slab_count), int(seq) & 0xFFFFFFFF, int(wait_ms)
    p.slab_stride = int(slab_stride)
    args = [flags.arg(), image.arg(L.IMAGE if image.arg_class == L.IMAGE else L.OUTPUT)] + [w.arg() for w in peer_wires]
    launch(stream, "gather_pull_u16", args, p)


# ------------------------------------------------------------------------------ maps ----------
def fused_map(stream: Stream, a: Buffer, x: Buffer, y: Buffer, out: Buffer, n: int) -> None:
    """out = tanh(a*x + y) * exp(-0.5*x*x) + sqrt(|y| + 1e-3), one kernel."""
    p = L.MapParams()
    p.size, p.n = C.sizeof(L.MapParams), int(n)
    launch(stream, "fused_map", [a.arg(L.INPUT), x.arg(L.INPUT), y.arg(L.INPUT), out.arg(L.OUTPUT)], p)


class Tape:
    """Builder for the ``map_tape`` operator: a fused chain of elementwise operations.

    >>> t = Tape(n_inputs=2)
    >>> v = t.op("tanh", t.op("add", t.input(0), t.input(1)))
    >>> t.output(v)
    """

    def __init__(self, n_inputs: int, row_vectors: Sequence[int] = (), col_vectors: Sequence[int] = (),
                 scalars: Sequence[int] = ()):
        self.n_inputs = n_inputs
        self.instr: list = []
        self.outputs: list = []
        self.row_mask = sum(1 << k for k in row_vectors)
        self.col_mask = sum(1 << k for k in col_vectors)
        self.scalar_mask = sum(1 << k for k in scalars)

    def input(self, k: int) -> int:
        if not 0 <= k < self.n_inputs:
            raise IndexError(k)
        return k

    def const(self, value: float) -> int:
        self.instr.append((L.T["const"], 0, 0, 0, float(value)))
        return self.n_inputs + len(self.instr) - 1

    def op(self, name: str, a: int, b: int = 0, c: int = 0) -> int:
        self.instr.append((L.T[name], a, b, c, 0.0))
        return self.n_inputs + len(self.instr) - 1

    def output(self, value: int, col_sum: bool = False) -> None:
        """Store ``value`` to the next output array; with ``col_sum`` the output array is a [cols] vector that
        receives the column sums of the value instead (the full-size value is never written)."""
        if col_sum:
            self.colsum_mask = getattr(self, "colsum_mask", 0) | (1 << len(self.outputs))
        self.outputs.append(value)

    def params(self, rows: int, cols: int) -> L.TapeParams:
        if len(self.instr) > L.TAPE_MAX_INSTR or len(self.outputs) > L.TAPE_MAX_OUTPUTS or self.n_inputs > L.TAPE_MAX_INPUTS:
            raise ValueError("tape exceeds the operator's limits")
        p = L.TapeParams()
        p.size = C.sizeof(L.TapeParams)
        p.n_inputs, p.n_outputs, p.n_instr = self.n_inputs, len(self.outputs), len(self.instr)
        p.rows, p.cols = int(rows), int(cols)
        p.row_vector_mask, p.col_vector_mask, p.scalar_mask = self.row_mask, self.col_mask, self.scalar_mask
        p.colsum_mask = getattr(self, "colsum_mask", 0)
        for k, v in enumerate(self.outputs):
            p.out_value[k] = v
        for k, (op, a, b, c, imm) in enumerate(self.instr):
            p.instr[k].op, p.instr[k].a, p.instr[k].b, p.instr[k].c, p.instr[k].imm = op, a, b, c, imm
        return p


def map_tape(stream: Stream, tape: Tape, inputs: Sequence[Buffer], outputs: Sequence[Buffer], rows: int, cols: int,
             interpret: bool = False) -> None:
    """Run the tape over [rows][cols] arrays as one kernel: compiled for this tape at first use, or, with
    ``interpret`` (and where no run-time compiler is installed), by the interpreting kernel.  Same bits either way."""
    args = [b.arg(L.INPUT) for b in inputs] + [b.arg(L.OUTPUT) for b in outputs]
    p = tape.params(rows, cols)
    if interpret:
        p.flags |= L.TAPE_FLAG_INTERPRET
    launch(stream, "map_tape", args, p)


def tape_jit_stats() -> dict:
    """Tapes compiled so far in this process and launches of compiled tapes."""
    a, b, cv, bv = C.c_uint64(), C.c_uint64(), C.c_int(), C.c_int()
    check(lib().vrhi_tape_jit_stats(C.byref(a), C.byref(b), C.byref(cv), C.byref(bv)))
    return {"compiled": a.value, "launches": b.value, "compiler_version": cv.value, "built_version": bv.value}


def tape_source(tape: Tape, rows: int = 4, cols: int = 4) -> str:
    """The CUDA source the library generates for this tape (no device needed)."""
    p = tape.params(rows, cols)
    need = C.c_uint64()
    check(lib().vrhi_tape_source(C.byref(p), None, 0, C.byref(need)))
    buf = C.create_string_buffer(need.value)
    check(lib().vrhi_tape_source(C.byref(p), buf, need.value, C.byref(need)))
    return buf.value.decode()


# ------------------------------------------------------------------------------ rows ----------
def _rows(rows: int, cols: int) -> L.RowsParams:
    p = L.RowsParams()
    p.size, p.rows, p.cols = C.sizeof(L.RowsParams), int(rows), int(cols)
    return p


def row_sum(stream: Stream, m: Buffer, out: Buffer, rows: int, cols: int) -> None:
    launch(stream, "row_sum", [m.arg(L.INPUT), out.arg(L.OUTPUT)], _rows(rows, cols))


def row_max(stream: Stream, m: Buffer, out: Buffer, rows: int, cols: int) -> None:
    launch(stream, "row_max", [m.arg(L.INPUT), out.arg(L.OUTPUT)], _rows(rows, cols))


def row_softmax(stream: Stream, m: Buffer, out: Buffer, rows: int, cols: int) -> None:
    launch(stream, "row_softmax", [m.arg(L.INPUT), out.arg(L.OUTPUT)], _rows(rows, cols))


def row_stats_softmax(stream: Stream, m: Buffer, out_sum: Buffer, out_max: Buffer, out_softmax: Buffer, rows: int,
                      cols: int) -> None:
    """Per-row sum, per-row max and softmax(row) from a single read of the matrix."""
    launch(stream, "row_stats_softmax",
           [m.arg(L.INPUT), out_sum.arg(L.OUTPUT), out_max.arg(L.OUTPUT), out_softmax.arg(L.OUTPUT)], _rows(rows, cols))


def col_sum(stream: Stream, m: Buffer, out: Buffer, rows: int, cols: int) -> None:
    launch(stream, "col_sum", [m.arg(L.INPUT), out.arg(L.OUTPUT)], _rows(rows, cols))


# ------------------------------------------------------------------------------ loss / grad ---
def _mse(rows: int, cols: int, denom: float) -> L.MseParams:
    p = L.MseParams()
    p.size, p.rows, p.cols, p.denom = C.sizeof(L.MseParams), int(rows), int(cols), float(denom)
    return p


def mse_tanh_fwd(stream: Stream, W: Buffer, x: Buffer, b: Buffer, t: Buffer, loss: Buffer, rows: int, cols: int,
                 denom: float = 0.0) -> None:
    """loss = sum((tanh(W*x + b) - t)^2) / denom over these rows (denom = 0: rows*cols)."""
    launch(stream, "mse_tanh_fwd", [W.arg(L.INPUT), x.arg(L.INPUT), b.arg(L.INPUT), t.arg(L.INPUT), loss.arg(L.OUTPUT)],
           _mse(rows, cols, denom))


def mse_tanh_bwd(stream: Stream, W: Buffer, x: Buffer, b: Buffer, t: Buffer, dW: Buffer, dx: Buffer, db: Buffer,
                 rows: int, cols: int, denom: float = 0.0, loss: Optional[Buffer] = None) -> None:
    """dW, dx (full size) and db (column sums) of the loss above, forward recomputed in the kernel."""
    args = [W.arg(L.INPUT), x.arg(L.INPUT), b.arg(L.INPUT), t.arg(L.INPUT), dW.arg(L.OUTPUT), dx.arg(L.OUTPUT),
            db.arg(L.OUTPUT)]
    if loss is not None:
        args.append(loss.arg(L.OUTPUT))
    launch(stream, "mse_tanh_bwd", args, _mse(rows, cols, denom))


def vertex_transform(stream: Stream, pos: Buffer, model: Buffer, view: Buffer, proj: Buffer, gl_position: Buffer,
                     varying: Buffer, n: int) -> None:
    """color.mlir:4-39 over an array of n vertices: gl_position = proj*(view*(model*(p,1))), varying = p."""
    p = L.MapParams()
    p.size, p.n = C.sizeof(L.MapParams), int(n)
    launch(stream, "vertex_transform", [pos.arg(L.INPUT), model.arg(L.UNIFORM), view.arg(L.UNIFORM), proj.arg(L.UNIFORM),
                                        gl_position.arg(L.OUTPUT), varying.arg(L.VARYING)], p)


def flat_color(stream: Stream, color: Buffer, fragments: Buffer, n: int) -> None:
    """color.mlir:43-59 over n fragments: every fragment = (c0, c1, c2, 1)."""
    p = L.MapParams()
    p.size, p.n = C.sizeof(L.MapParams), int(n)
    launch(stream, "flat_color", [color.arg(L.UNIFORM), fragments.arg(L.IMAGE)], p)


def fp32_probe(stream: Stream, out: Buffer, ffma_per_thread: int, threads: int = 0, variant: int = 0) -> None:
    """``variant``: 0 scalar fma, 1 packed fma.rn.f32x2, 2 packed with an integer add per fma, 3 scalar with one."""
    p = L.ProbeParams()
    p.size, p.ffma_per_thread, p.threads, p.variant = C.sizeof(L.ProbeParams), int(ffma_per_thread), int(threads), int(variant)
    launch(stream, "fp32_probe", [out.arg(L.OUTPUT)], p)


# ------------------------------------------------------------------------------ partitioning --
def partition_rows(total_rows: int, world: int, rank: int, scheme: int = L.PART_CYCLIC, chunk_rows: int = 128) -> L.RowPartition:
    out = L.RowPartition()
    check(lib().vrhi_partition_rows(int(total_rows), int(chunk_rows), int(world), int(rank), int(scheme), C.byref(out)))
    return out


def partition_leading(n: int, world: int, rank: int):
    b, c = C.c_uint64(), C.c_uint64()
    check(lib().vrhi_partition_leading(int(n), int(world), int(rank), C.byref(b), C.byref(c)))
    return b.value, c.value
