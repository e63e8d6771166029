"""Python face of the C++ execution graph (``vrhi_graph_*``): build, differentiate, fuse, launch.

All planning (fusion of elementwise chains into single kernels, reverse-mode differentiation,
kernel selection) happens inside ``libvrhi.so``; this file only forwards node construction and
offers operator overloading on node handles.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _lib as L
from ._lib import check, lib
from .rhi import Buffer, Device, Stream


class Node:
    __slots__ = ("g", "id")

    def __init__(self, g: "Graph", node_id: int):
        self.g, self.id = g, node_id

    def _bin(self, op, other, swap=False):
        o = other if isinstance(other, Node) else self.g.const(float(other))
        a, b = (o, self) if swap else (self, o)
        return self.g.binary(op, a, b)

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __truediv__(self, o): return self._bin("div", o)
    def __rtruediv__(self, o): return self._bin("div", o, True)
    def __neg__(self): return self.g.unary("neg", self)
    def __abs__(self): return self.g.unary("abs", self)


class Graph:
    """A tensor graph over one [rows][cols] problem shape on one device."""

    def __init__(self, dev: Device, rows: int, cols: int, specialize: bool = True):
        h = C.c_void_p()
        check(lib().vrhi_graph_create(dev._h, int(rows), int(cols), C.byref(h)))
        self._h, self.dev, self.rows, self.cols = h, dev, rows, cols
        self._keep: list = []
        if not specialize:
            check(lib().vrhi_graph_set_flags(self._h, 1))

    def close(self) -> None:
        if self._h:
            lib().vrhi_graph_destroy(self._h)
            self._h = None

    def _node(self, fn, *args) -> Node:
        v = C.c_int()
        check(fn(self._h, *args, C.byref(v)))
        return Node(self, v.value)

    def input(self, buf: Buffer, shape: int = L.SHAPE_FULL) -> Node:
        self._keep.append(buf)
        return self._node(lib().vrhi_graph_input, buf._h, int(shape))

    def const(self, value: float) -> Node:
        return self._node(lib().vrhi_graph_const, C.c_float(value))

    def unary(self, op: str, a: Node) -> Node:
        return self._node(lib().vrhi_graph_unary, L.T[op], a.id)

    def binary(self, op: str, a: Node, b: Node) -> Node:
        return self._node(lib().vrhi_graph_binary, L.T[op], a.id, b.id)

    def reduce(self, op: int, a: Node) -> Node:
        return self._node(lib().vrhi_graph_reduce, int(op), a.id)

    def row_sum(self, a): return self.reduce(L.R_ROW_SUM, a)
    def row_max(self, a): return self.reduce(L.R_ROW_MAX, a)
    def col_sum(self, a): return self.reduce(L.R_COL_SUM, a)
    def sum(self, a): return self.reduce(L.R_SUM_ALL, a)
    def mean(self, a): return self.reduce(L.R_MEAN_ALL, a)

    def softmax(self, a: Node) -> Node:
        return self._node(lib().vrhi_graph_softmax, a.id)

    def tanh(self, a): return self.unary("tanh", a)
    def exp(self, a): return self.unary("exp", a)
    def sqrt(self, a): return self.unary("sqrt", a)
    def square(self, a): return self.unary("square", a)
    def log(self, a): return self.unary("log", a)

    def grad(self, loss: Node, wrt: Sequence[Node]) -> list:
        ids = (C.c_int * len(wrt))(*[w.id for w in wrt])
        out = (C.c_int * len(wrt))()
        check(lib().vrhi_graph_grad(self._h, loss.id, ids, len(wrt), out))
        return [Node(self, out[k]) for k in range(len(wrt))]

    def output(self, node: Node, buf: Buffer) -> None:
        self._keep.append(buf)
        check(lib().vrhi_graph_output(self._h, node.id, buf._h))

    def compile(self) -> None:
        check(lib().vrhi_graph_compile(self._h))

    def launch(self, stream: Stream) -> None:
        check(lib().vrhi_graph_launch(self._h, stream._h))

    def describe(self) -> str:
        need = C.c_size_t()
        check(lib().vrhi_graph_describe(self._h, None, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value)
        check(lib().vrhi_graph_describe(self._h, buf, need.value, None))
        return buf.value.decode()

    def kernel_count(self) -> int:
        v = C.c_int()
        check(lib().vrhi_graph_kernel_count(self._h, C.byref(v)))
        return v.value
