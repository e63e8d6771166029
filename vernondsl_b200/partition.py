"""Single-box multi-GPU partitioner: one process per GPU, ``torch.distributed`` for the exchange.

Work is split by the planner inside ``libvrhi.so`` (``vrhi_partition_rows`` /
``vrhi_partition_leading``); this module adds the only exchange steps the path has:

* escape-time images: every rank computes its own row chunks into a full-size image at their
  true position, then the chunks are all-gathered in place (no staging copy, no permutation);
* the tanh-MSE backward: ``db`` and the loss are all-reduced (sum); ``dW`` and ``dx`` stay sharded.

Map and row operators need no exchange: each rank owns a slice of the leading axis.
Collectives run on tensors that alias the library's buffers, on whatever backend the process
group was created with (NCCL on GPUs; gloo in the CPU tests of this logic).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np

from . import _lib as L
from . import ops


@dataclass(frozen=True)
class ImagePlan:
    """Row ownership of one rank for an image of ``height`` rows."""
    height: int
    world: int
    rank: int
    scheme: int
    part: L.RowPartition

    def chunks(self) -> List[Tuple[int, int]]:
        """(first_row, n_rows) of every chunk this rank owns, in launch order."""
        p, out = self.part, []
        for k in range(p.chunk_count):
            c = p.chunk_first + k * p.chunk_step
            r0 = c * p.chunk_rows
            out.append((r0, min(self.height, r0 + p.chunk_rows) - r0))
        return out


def plan_image(height: int, world: int, rank: int, scheme: int = L.PART_CYCLIC, chunk_rows: int = 128) -> ImagePlan:
    """Cyclic chunks by default: escape-time cost varies smoothly over the image, so dealing
    128-row chunks round-robin balances ranks where equal contiguous bands do not."""
    return ImagePlan(height, world, rank, scheme, ops.partition_rows(height, world, rank, scheme, chunk_rows))


def owner_of_row(plan: ImagePlan, row: int) -> int:
    """Rank that computes image row ``row`` under ``plan``'s scheme (the same for every rank)."""
    c = row // plan.part.chunk_rows
    return c % plan.world if plan.scheme == L.PART_CYCLIC else c


def all_gather_image(image, plan: ImagePlan, group=None, async_op: bool = False, slab_range=None):
    """All-gather the row chunks of ``image`` (a [height, width] tensor holding this rank's chunks
    at their true rows) so that every rank ends with the whole image.

    Cyclic plans whose chunk count divides evenly gather IN PLACE: the image viewed as
    [slab, rank, chunk_rows*width] already has rank r's data at [:, r, :], which is exactly the
    output layout of an all-gather of each slab.  Anything else falls back to one broadcast per
    chunk from its owner.  ``slab_range=(lo, hi)`` restricts an even cyclic gather to slabs lo..hi-1
    (slab k holds chunks k*world .. k*world+world-1), so that the gather of finished slabs can overlap
    the computation of later ones.  Returns the list of work handles when ``async_op``.
    """
    import torch.distributed as dist

    world, p = plan.world, plan.part
    if world == 1:
        return []
    height, width = image.shape
    works = []
    n_chunks = -(-height // p.chunk_rows)
    even = plan.scheme == L.PART_CYCLIC and height % p.chunk_rows == 0 and n_chunks % world == 0
    if even:
        slabs = image.view(n_chunks // world, world, p.chunk_rows * width)
        lo, hi = slab_range if slab_range is not None else (0, slabs.shape[0])
        if image.is_cuda and hasattr(dist, "_coalescing_manager") and hi - lo > 1:
            # one NCCL group for all slabs: a single launch instead of one per slab
            with dist._coalescing_manager(group=group, device=image.device, async_ops=True) as cm:
                for k in range(lo, hi):
                    dist.all_gather_into_tensor(slabs[k].view(-1), slabs[k, plan.rank], group=group)
            if async_op:
                works.append(cm)
            else:
                cm.wait()
        else:
            for k in range(lo, hi):
                w = dist.all_gather_into_tensor(slabs[k].view(-1), slabs[k, plan.rank], group=group, async_op=async_op)
                if async_op:
                    works.append(w)
    else:
        for c in range(n_chunks):
            r0 = c * p.chunk_rows
            r1 = min(height, r0 + p.chunk_rows)
            src = c % world if plan.scheme == L.PART_CYCLIC else c  # contiguous: chunk c is rank c's band
            src_global = dist.get_global_rank(group, src) if group is not None else src
            w = dist.broadcast(image[r0:r1], src=src_global, group=group, async_op=async_op)
            if async_op:
                works.append(w)
    return works


def all_reduce_sum(tensors, group=None) -> None:
    """Sum small per-rank partials (db, loss, reduction partials) across ranks, in place."""
    import torch.distributed as dist

    if dist.get_world_size(group) == 1:
        return
    for t in tensors:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


def leading_slice(n: int, world: int, rank: int) -> Tuple[int, int]:
    """(begin, count) of this rank's share of a leading axis of length n."""
    return ops.partition_leading(n, world, rank)


class PeerImageExchange:
    """All-gather of an image's row chunks by peer copies instead of a collective kernel.

    Every rank maps every other rank's image (CUDA IPC inside one box) and pushes its own chunks
    into them with strided device-to-device copies: chunks of one rank lie ``world`` chunks apart, so
    one 2-D copy per peer moves a whole range of slabs.  The copy engines carry the data over
    NVLink without occupying SMs, so pushes of finished slabs overlap the kernel computing the
    next ones.  ``finish`` orders a one-element all-reduce after this rank's pushes: when it
    completes, every peer's pushes into this rank's image have completed too.

    Needs an even cyclic plan (the in-place layout of :func:`all_gather_image`) and an image buffer
    allocated by the library (``Device.empty``); anything else should use :func:`all_gather_image`.
    """

    def __init__(self, dev, image, plan: ImagePlan, row_bytes: int, group=None):
        import torch
        import torch.distributed as dist

        p = plan.part
        n_chunks = -(-plan.height // p.chunk_rows)
        if not (plan.scheme == L.PART_CYCLIC and plan.height % p.chunk_rows == 0 and n_chunks % plan.world == 0):
            raise ValueError("peer exchange needs a cyclic plan whose chunk count divides evenly")
        self.image, self.plan, self.group = image, plan, group
        self.chunk_bytes = p.chunk_rows * row_bytes
        self.n_slabs = n_chunks // plan.world
        handles = [None] * plan.world
        dist.all_gather_object(handles, image.ipc_handle(), group=group)
        self.peers = {r: dev.open_ipc(handles[r], image.nbytes, L.IMAGE) for r in range(plan.world) if r != plan.rank}
        self._flag = torch.zeros(1, device=f"cuda:{dev.ordinal}")

    def push(self, stream, slab_range=None) -> None:
        """Enqueue the copies of this rank's chunks of slabs lo..hi-1 into every peer.  ``stream`` is one
        stream, or a list with one stream per peer so that the pushes to different peers run on
        different copy engines at the same time."""
        lo, hi = slab_range if slab_range is not None else (0, self.n_slabs)
        if hi <= lo:
            return
        world, rank = self.plan.world, self.plan.rank
        offset = (lo * world + rank) * self.chunk_bytes
        pitch = world * self.chunk_bytes
        # start with the next rank so that, at any moment, the ranks write to different peers
        streams = stream if isinstance(stream, (list, tuple)) else [stream] * (world - 1)
        for step in range(1, world):
            peer = self.peers[(rank + step) % world]
            self.image.copy_2d_to(peer, offset, pitch, offset, pitch, self.chunk_bytes, hi - lo, streams[step - 1])

    def finish(self, torch_stream) -> None:
        """Stream-ordered completion: after this, all ranks' pushes are visible in this rank's image."""
        import torch
        import torch.distributed as dist

        with torch.cuda.stream(torch_stream):
            dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        for b in self.peers.values():
            b.close()
        self.peers = {}


class WireImageExchange:
    """The same gather with uint16 counts on the wire: half the bytes cross NVLink.

    The escape-time kernel writes every count twice, as uint32 into the rank's image and as uint16
    into a wire image of the same geometry (``ops.escape_time(..., wire=exchange.wire)``).  The wire
    chunks are pushed into the peers' wire images by the copy engines (:class:`PeerImageExchange`);
    ``finish`` orders the one-element all-reduce behind the pushes and then widens the peers' rows
    from the local wire image into the uint32 image (``widen_rows_u16``, HBM-bound).  Needs
    ``max_iter <= 65535``, so that nothing is lost.
    """

    def __init__(self, dev, image, plan: ImagePlan, width: int, group=None):
        self.dev, self.image, self.plan, self.width = dev, image, plan, int(width)
        self.wire = dev.empty((plan.height, self.width), np.uint16, L.IMAGE)
        self.peer = PeerImageExchange(dev, self.wire, plan, self.width * 2, group)
        self.n_slabs = self.peer.n_slabs

    def push(self, stream, slab_range=None) -> None:
        self.peer.push(stream, slab_range)

    def finish(self, torch_stream, stream, slab_range=None) -> None:
        """``torch_stream`` and ``stream`` are the same CUDA stream (torch's handle for the collective,
        the library's for the kernel).  After this, stream-ordered, the uint32 image holds every rank's
        rows of ``slab_range`` (default: all)."""
        from . import ops

        self.peer.finish(torch_stream)
        lo, hi = slab_range if slab_range is not None else (0, self.n_slabs)
        p = self.plan
        ops.widen_rows_u16(stream, self.wire, self.image, self.width, p.height, p.part.chunk_rows, p.world, p.rank, lo, hi - lo)

    def close(self) -> None:
        self.peer.close()
        self.wire.close()
