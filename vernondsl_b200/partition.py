"""Single-box multi-GPU partitioner: one process per GPU.

Work is split by the planner inside ``libvrhi.so`` (``vrhi_partition_rows`` /
``vrhi_partition_leading``).  The exchange steps the path has, the gather of an escape-time
image and the sum of ``db`` and the loss of a row-sharded backward, are the library's own
(``vrhi_exchange_*`` and ``vrhi_group_all_reduce_sum_f32``, bound in :mod:`vernondsl_b200.group`).
This module holds the planning helpers around them and three alternative forms of the image
gather, kept for comparison; they run over ``torch.distributed``:

* :func:`all_gather_image`: in-place all-gather of the row chunks with the process group's
  backend (NCCL on GPUs; gloo in the CPU tests of this logic);
* :class:`PeerImageExchange`: uint32 rows pushed into the peers' images by the copy engines;
* :class:`PullImageExchange`: each rank reads its peers' uint16 rows over NVLink and widens them
  in the same kernel.

Map and row operators need no exchange: each rank owns a slice of the leading axis.
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


def comb_groups(plan: ImagePlan, groups: int) -> List[Tuple[Tuple[int, int, int], Tuple[int, int, int]]]:
    """Split a cyclic plan's slabs into ``groups`` combs for a pipelined step: comb g takes slabs g, g+groups,
    g+2*groups, ...  Every comb reaches over the whole image, so the combs cost about the same although rows
    near the set cost many times the rows at the edges.  Returns, per non-empty comb,
    ``((chunk_first, chunk_step, chunk_count), (slab_first, slab_count, slab_stride))``: the first triple goes
    into the escape-time parameters of the comb's launch, the second names the comb to the exchange."""
    if plan.scheme != L.PART_CYCLIC:
        raise ValueError("combs are defined for cyclic plans")
    if groups < 1:
        raise ValueError("at least one group")
    p, out = plan.part, []
    for g in range(groups):
        count = (p.chunk_count - g + groups - 1) // groups if g < p.chunk_count else 0
        if count > 0:
            out.append(((p.chunk_first + g * p.chunk_step, p.chunk_step * groups, count), (g, count, groups)))
    return out


def owner_of_row(plan: ImagePlan, row: int) -> int:
    """Rank that computes image row ``row`` under ``plan``'s scheme (the same for every rank)."""
    c = row // plan.part.chunk_rows
    return c % plan.world if plan.scheme == L.PART_CYCLIC else c


def all_gather_image(image, plan: ImagePlan, group=None, async_op: bool = False, slab_range=None, slabs=None):
    """All-gather the row chunks of ``image`` (a [height, width] tensor holding this rank's chunks
    at their true rows) so that every rank ends with the whole image.

    Cyclic plans whose chunk count divides evenly gather IN PLACE: the image viewed as
    [slab, rank, chunk_rows*width] already has rank r's data at [:, r, :], which is exactly the
    output layout of an all-gather of each slab.  Anything else falls back to one broadcast per
    chunk from its owner.  ``slab_range=(lo, hi)`` restricts an even cyclic gather to slabs lo..hi-1
    (slab k holds chunks k*world .. k*world+world-1), ``slabs=(first, count, stride)`` to slabs
    first + k*stride, so that the gather of finished slabs can overlap the computation of later ones.  Returns the list of work handles when ``async_op``.
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
        slab_view = image.view(n_chunks // world, world, p.chunk_rows * width)
        if slabs is not None:
            which = range(slabs[0], slabs[0] + slabs[1] * slabs[2], slabs[2])
        else:
            lo, hi = slab_range if slab_range is not None else (0, slab_view.shape[0])
            which = range(lo, hi)
        slabs = slab_view
        if image.is_cuda and hasattr(dist, "_coalescing_manager") and len(which) > 1:
            # one NCCL group for all slabs: a single launch instead of one per slab
            with dist._coalescing_manager(group=group, device=image.device, async_ops=True) as cm:
                for k in which:
                    dist.all_gather_into_tensor(slabs[k].view(-1), slabs[k, plan.rank], group=group)
            if async_op:
                works.append(cm)
            else:
                cm.wait()
        else:
            for k in which:
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

    The pushes land in the peers' images themselves.  A rank must therefore not start the pushes of
    a step before every peer is done reading the image of the step before: order them behind a
    collective (or barrier) issued after those reads.  The library's own exchange
    (:class:`vernondsl_b200.group.Exchange`) needs no such care: it sends through two alternating
    wire images.
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

    def push(self, stream, slabs=None) -> None:
        """Enqueue the copies of this rank's chunks of slabs ``first + k*stride`` (k < count) into every peer;
        ``slabs`` = (first, count, stride), default all.  ``stream`` is one stream, or a list with one stream per
        peer so that the pushes to different peers run on different copy engines at the same time."""
        first, count, stride = slabs if slabs is not None else (0, self.n_slabs, 1)
        if count <= 0:
            return
        world, rank = self.plan.world, self.plan.rank
        offset = (first * world + rank) * self.chunk_bytes
        pitch = world * stride * self.chunk_bytes
        # start with the next rank so that, at any moment, the ranks write to different peers
        streams = stream if isinstance(stream, (list, tuple)) else [stream] * (world - 1)
        for step in range(1, world):
            peer = self.peers[(rank + step) % world]
            self.image.copy_2d_to(peer, offset, pitch, offset, pitch, self.chunk_bytes, count, streams[step - 1])

    def finish(self, torch_stream) -> None:
        """Stream-ordered completion: after this, every rank's pushes enqueued before its matching call
        are visible in this rank's image."""
        import torch
        import torch.distributed as dist

        with torch.cuda.stream(torch_stream):
            dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        for b in self.peers.values():
            b.close()
        self.peers = {}


class PullImageExchange:
    """The gather in pull form: every rank reads its peers' uint16 rows out of their memory over
    NVLink and widens them into its own uint32 image in the same kernel (``gather_pull_u16``).

    Nothing is pushed and no collective runs: after computing a group of slabs (with
    ``ops.escape_time(..., wire=exchange.wire)``) a rank calls ``signal``, which stores the group's
    sequence number into its slot of every peer's flag array; ``pull`` waits (bounded, on the
    device) until every peer's slot has reached that number and then copies.  Two wire images
    alternate from step to step so that a rank never overwrites rows a slower peer is still reading.

    ``groups`` is the number of signal/pull pairs per step and must be the same on every rank.
    """

    def __init__(self, dev, image, plan: ImagePlan, width: int, groups: int, group=None, wait_ms: int = 2000):
        import torch.distributed as dist

        p = plan.part
        n_chunks = -(-plan.height // p.chunk_rows)
        if not (plan.scheme == L.PART_CYCLIC and plan.height % p.chunk_rows == 0 and n_chunks % plan.world == 0):
            raise ValueError("the pull exchange needs a cyclic plan whose chunk count divides evenly")
        if not 2 <= plan.world <= L.GATHER_MAX_WORLD:
            raise ValueError(f"the pull exchange serves 2..{L.GATHER_MAX_WORLD} ranks")
        if width % 8:
            raise ValueError("the pull exchange needs a width that is a multiple of 8 pixels")
        self.dev, self.image, self.plan, self.width = dev, image, plan, int(width)
        self.groups, self.wait_ms = int(groups), int(wait_ms)
        self.n_slabs = n_chunks // plan.world
        self.wires = [dev.empty((plan.height, self.width), np.uint16, L.IMAGE) for _ in range(2)]
        self.flags = dev.empty((1 << 19,), np.uint32, L.STORAGE_BUFFER)   # its own 2 MiB allocation; world slots are used
        self.flags.fill(0)
        dev.synchronize()
        mine = (self.wires[0].ipc_handle(), self.wires[1].ipc_handle(), self.flags.ipc_handle())
        handles = [None] * plan.world
        dist.all_gather_object(handles, mine, group=group)
        self.peer_wires = [[dev.open_ipc(handles[r][b], self.wires[b].nbytes, L.STORAGE_BUFFER) for r in range(plan.world) if r != plan.rank]
                           for b in range(2)]
        self.peer_flags = [dev.open_ipc(handles[r][2], self.flags.nbytes, L.STORAGE_BUFFER) for r in range(plan.world) if r != plan.rank]
        self.step = 0
        dist.barrier(group=group)   # every rank has zeroed its flags before anyone signals

    @property
    def wire(self):
        """The wire image this step's kernels write into."""
        return self.wires[self.step & 1]

    def next_step(self) -> None:
        self.step += 1

    def _seq(self, g: int) -> int:
        return self.step * self.groups + g + 1

    def signal(self, stream, g: int) -> None:
        """Enqueue on ``stream`` (behind the kernels that computed group ``g``) the ready mark for the peers.
        Precondition: this rank's pulls of the step before the previous one are ordered before this call on the
        GPU (the two wire images alternate, so the kernels of this step overwrite the rows the peers pulled two
        steps ago; a peer can be at most one step behind, because this rank's pulls waited for its signals)."""
        ops.gather_signal(stream, self.peer_flags, self.plan.world, self.plan.rank, self._seq(g))

    def pull(self, stream, g: int, slabs) -> None:
        first, count, stride = slabs
        p = self.plan
        ops.gather_pull_u16(stream, self.flags, self.image, self.peer_wires[self.step & 1], self.width, p.height, p.part.chunk_rows,
                            p.world, p.rank, first, count, self._seq(g), self.wait_ms, stride)

    def close(self) -> None:
        for b in self.peer_flags + self.peer_wires[0] + self.peer_wires[1]:
            b.close()
        self.peer_flags, self.peer_wires = [], [[], []]
        for b in self.wires + [self.flags]:
            b.close()
