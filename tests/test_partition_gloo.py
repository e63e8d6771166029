"""CPU, world_size 2 and 3 over gloo: the multi-GPU partitioner's exchange logic (in-place chunk
all-gather of an image, all-reduce of gradient partials) with CPU tensors standing in for device
buffers.  No kernel runs here; ranks fill their own rows with a known pattern."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vernondsl_b200 import _lib as L
from vernondsl_b200 import partition


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, height, width, scheme, chunk, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = partition.plan_image(height, world, rank, scheme, chunk)
        image = torch.full((height, width), -1, dtype=torch.int32)
        for r0, n in plan.chunks():
            for r in range(r0, r0 + n):
                assert partition.owner_of_row(plan, r) == rank
                image[r] = torch.arange(width, dtype=torch.int32) + 1000 * r
        works = partition.all_gather_image(image, plan, async_op=True)
        for w in works:
            w.wait()
        want = torch.arange(width, dtype=torch.int32)[None, :] + 1000 * torch.arange(height, dtype=torch.int32)[:, None]
        ok_image = bool(torch.equal(image, want))
        # gradient partials: db and loss add across ranks
        db = torch.full((16,), float(rank + 1))
        loss = torch.tensor([0.5 * (rank + 1)])
        partition.all_reduce_sum([db, loss])
        tot = world * (world + 1) / 2
        ok_sum = bool(torch.allclose(db, torch.full((16,), tot)) and abs(loss.item() - 0.5 * tot) < 1e-6)
        b, c = partition.leading_slice(1000003, world, rank)
        np.save(os.path.join(result_dir, f"r{rank}.npy"), np.array([ok_image, ok_sum, b, c], dtype=np.int64))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,height,width,scheme,chunk", [
    (2, 64, 8, L.PART_CYCLIC, 8),      # even: in-place all-gather of slabs
    (2, 70, 5, L.PART_CYCLIC, 8),      # ragged last chunk: broadcast per chunk
    (3, 64, 4, L.PART_CYCLIC, 8),      # chunk count not a multiple of the world size
    (2, 33, 6, L.PART_CONTIGUOUS, 0),  # one band per rank
])
def test_image_gather_and_partial_sums(tmp_path, world, height, width, scheme, chunk):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, height, width, scheme, chunk, str(tmp_path)), nprocs=world, join=True)
    spans = []
    for r in range(world):
        ok_image, ok_sum, b, c = np.load(tmp_path / f"r{r}.npy")
        assert ok_image and ok_sum
        spans.append((b, c))
    assert spans[0][0] == 0 and sum(c for _, c in spans) == 1000003


@pytest.mark.parametrize("world,slabs,groups", [(2, 6, 3), (4, 8, 4), (3, 5, 2), (2, 3, 8), (1, 7, 4)])
def test_combs_cover_every_owned_chunk_exactly_once(world, slabs, groups):
    chunk, height = 4, 4 * world * slabs
    for rank in range(world):
        plan = partition.plan_image(height, world, rank, L.PART_CYCLIC, chunk)
        owned = [r0 // chunk for r0, _ in plan.chunks()]
        seen, slabs_seen = [], []
        for (first, step, count), (s0, n, stride) in partition.comb_groups(plan, groups):
            assert count == n and stride == groups
            seen += [first + k * step for k in range(count)]
            slabs_seen += [s0 + k * stride for k in range(n)]
        assert sorted(seen) == owned
        assert sorted(slabs_seen) == list(range(slabs))
        # chunk ids and slab ids name the same rows: chunk = slab * world + rank
        assert sorted(seen) == sorted(s * world + rank for s in slabs_seen)
    with pytest.raises(ValueError):
        partition.comb_groups(partition.plan_image(height, world, 0, L.PART_CONTIGUOUS, 0), 2)


def _comb_worker(rank, world, port, height, width, chunk, groups, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = partition.plan_image(height, world, rank, L.PART_CYCLIC, chunk)
        image = torch.full((height, width), -1, dtype=torch.int32)
        want = torch.arange(width, dtype=torch.int32)[None, :] + 1000 * torch.arange(height, dtype=torch.int32)[:, None]
        ok_partial = True
        done_slabs = set()
        for (first, step, count), comb in partition.comb_groups(plan, groups):
            for k in range(count):                      # "compute" this comb's chunks
                r0 = (first + k * step) * chunk
                image[r0:r0 + chunk] = want[r0:r0 + chunk]
            partition.all_gather_image(image, plan, slabs=comb)
            done_slabs |= {comb[0] + k * comb[2] for k in range(comb[1])}
            for s in range(height // (chunk * world)):  # gathered combs are whole, the others still hold only own rows
                rows = slice(s * world * chunk, (s + 1) * world * chunk)
                if s in done_slabs:
                    ok_partial &= bool(torch.equal(image[rows], want[rows]))
        np.save(os.path.join(result_dir, f"c{rank}.npy"), np.array([ok_partial, bool(torch.equal(image, want))], dtype=np.int64))
    finally:
        dist.destroy_process_group()


def test_gather_comb_by_comb_over_gloo(tmp_path):
    world, height, width, chunk, groups = 2, 96, 5, 8, 3
    mp.spawn(_comb_worker, args=(world, _free_port(), height, width, chunk, groups, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok_partial, ok_all = np.load(tmp_path / f"c{r}.npy")
        assert ok_partial and ok_all
