"""Groups of GPUs: binding of ``vrhi_group_*`` and ``vrhi_exchange_*`` (``include/vrhi.h``).

One rank per GPU of one box.  The library needs one service from its caller, an all-gather of
small byte records, and only while a group or an exchange is created; :func:`torch_allgather`
supplies it from a ``torch.distributed`` process group (any backend), but a pipe, MPI or a
key-value store does as well.  Every step after that runs inside ``libvrhi.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional

from . import _lib as L
from ._lib import check, lib
from .rhi import Buffer, Device, Stream


def torch_allgather(group=None) -> Callable[[bytes], List[bytes]]:
    """An all-gather of byte strings over a ``torch.distributed`` process group."""
    import torch.distributed as dist

    def gather(record: bytes) -> List[bytes]:
        out = [None] * dist.get_world_size(group)
        dist.all_gather_object(out, record, group=group)
        return out

    return gather


class Group:
    """``vrhi_group``: this rank's membership of a group of ``world`` ranks.

    ``allgather(record: bytes) -> list of world byte strings in rank order`` is the caller's
    bootstrap service (unused when ``world == 1``)."""

    def __init__(self, dev: Device, world: int, rank: int, allgather: Optional[Callable[[bytes], List[bytes]]] = None):
        self.dev, self.world, self.rank = dev, int(world), int(rank)
        self._error = None

        def trampoline(_user, send, recv, nbytes):
            try:
                parts = allgather(C.string_at(send, nbytes))
                if len(parts) != self.world or any(len(p) != nbytes for p in parts):
                    raise ValueError("the all-gather must return one record of the same size per rank")
                C.memmove(recv, b"".join(parts), nbytes * self.world)
                return 0
            except Exception as exc:  # an exception must not cross the C boundary
                self._error = exc
                return 1

        self._cb = L.ALLGATHER_FN(trampoline) if allgather is not None else C.cast(None, L.ALLGATHER_FN)
        h = C.c_void_p()
        self._guard(lib().vrhi_group_create(dev._h, self.world, self.rank, self._cb, None, C.byref(h)))
        self._h = h

    def _guard(self, status: int) -> None:
        if status != L.OK and self._error is not None:
            err, self._error = self._error, None
            raise err
        check(status)

    def set_wait_ms(self, wait_ms: int) -> None:
        check(lib().vrhi_group_set_wait_ms(self._h, int(wait_ms)))

    def all_reduce_sum(self, buf: Buffer, n: int, stream: Stream, offset: int = 0) -> None:
        """Sum ``n`` floats (at most 16384) of ``buf`` over the ranks, in place, on ``stream``."""
        check(lib().vrhi_group_all_reduce_sum_f32(self._h, buf._h, int(offset), int(n), stream._h))

    def image_exchange(self, image: Buffer, width: int, height: int, chunk_rows: int) -> "Exchange":
        return Exchange(self, image, width, height, chunk_rows)

    def close(self) -> None:
        if self._h:
            check(lib().vrhi_group_destroy(self._h))
            self._h = None


class _Borrowed(Buffer):
    """A buffer the library owns (closing it here does nothing)."""

    def close(self) -> None:
        self._h = None


class Exchange:
    """``vrhi_exchange``: the gather of an escape-time image computed in cyclic row chunks."""

    def __init__(self, group: Group, image: Buffer, width: int, height: int, chunk_rows: int):
        self.group, self.image, self.width, self.height, self.chunk_rows = group, image, int(width), int(height), int(chunk_rows)
        h = C.c_void_p()
        group._guard(lib().vrhi_exchange_create(group._h, image._h, self.width, self.height, self.chunk_rows, C.byref(h)))
        self._h = h

    @property
    def planes(self):
        """``(wire, bytes)``: the uint16 wire image and the byte plane this step's ``escape_time`` launches write
        beside the image (``ops.escape_time(..., wire=wire, byte_plane=bytes)``); ``bytes`` is None where the
        exchange does not squeeze the counts."""
        w, b = C.c_void_p(), C.c_void_p()
        check(lib().vrhi_exchange_planes(self._h, C.byref(w), C.byref(b)))
        n = self.width * self.height
        return (_Borrowed(self.group.dev, w, 2 * n, L.IMAGE), _Borrowed(self.group.dev, b, n, L.IMAGE) if b.value else None)

    def publish(self, compute_stream: Stream, slabs) -> None:
        """``slabs`` = (first, count, stride): the slabs the launches enqueued on ``compute_stream`` computed."""
        first, count, stride = slabs
        check(lib().vrhi_exchange_publish(self._h, compute_stream._h, int(first), int(count), int(stride)))

    def complete(self, stream: Stream) -> None:
        check(lib().vrhi_exchange_complete(self._h, stream._h))

    def check(self) -> None:
        check(lib().vrhi_exchange_check(self._h))

    def launch_count(self) -> int:
        v = C.c_uint64()
        check(lib().vrhi_exchange_launch_count(self._h, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._h:
            check(lib().vrhi_exchange_destroy(self._h))
            self._h = None
