"""One rank of the multi-GPU gather test (launched by test_multi_gpu.py through torch.distributed.run).

Every rank computes its comb of chunks of a small Julia image, the image is gathered with each
exchange in turn (the library's own first among them), and every rank compares its whole image with
the CPU oracle."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    import torch
    import torch.distributed as dist

    import oracle
    import vernondsl_b200 as vd
    from vernondsl_b200 import _lib as L
    from vernondsl_b200 import ops, partition

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    dev = vd.Device(local)
    W, chunk_rows, slabs, G = 512, 16, 6, 3
    H = chunk_rows * world * slabs
    max_iter = 600
    dx, dy = ops.grid_steps(-1.6, 1.6, -1.6, 1.6, W, H)
    want, _ = oracle.escape_time(oracle.JULIA, W, H, -1.6, -1.6, dx, dy, -0.8, 0.156, max_iter)
    plan = partition.plan_image(H, world, rank, L.PART_CYCLIC, chunk_rows)
    tstream, cstream = torch.cuda.Stream(device=local), torch.cuda.Stream(device=local)
    st, cst = dev.wrap_stream(tstream.cuda_stream), dev.wrap_stream(cstream.cuda_stream)
    image = dev.empty((H, W), np.uint32, L.IMAGE)
    image_t = image.as_tensor(np.uint32, (H, W))
    base = ops.escape_params(L.JULIA, W, H, -1.6, -1.6, dx, dy, cr=-0.8, ci=0.156, max_iter=max_iter, partition=plan.part)
    failures = []

    def groups():
        import copy
        for g, ((first, step, count), comb) in enumerate(partition.comb_groups(plan, G)):
            p = copy.copy(base)
            p.chunk_first, p.chunk_step, p.chunk_count = first, step, count
            yield g, p, comb

    def check(name):
        torch.cuda.synchronize()
        st.check()
        cst.check()
        got = image.download(dtype=np.uint32, shape=(H, W))
        if not np.array_equal(got, want):
            failures.append(f"{name}: {int((got != want).sum())} pixels differ on rank {rank}")
        image.fill(0xEE)
        dev.synchronize()
        dist.barrier()

    # NCCL all-gather, comb by comb
    for g, p, comb in groups():
        ops.escape_time(st, image, p)
        cstream.wait_stream(tstream)
        with torch.cuda.stream(cstream):
            partition.all_gather_image(image_t, plan, slabs=comb)
    check("nccl")

    # uint32 rows pushed by the copy engines
    ex = partition.PeerImageExchange(dev, image, plan, W * 4)
    for g, p, comb in groups():
        ops.escape_time(st, image, p)
        cstream.wait_stream(tstream)
        ex.push(cst, comb)
    ex.finish(cstream)
    check("p2p")
    ex.close()

    # the library's own exchange (vrhi_exchange_*): uint16 rows stored into the peers, sequence flags, two wire
    # images in turn.  Three steps with a different constant each, back to back: no host synchronisation and no
    # barrier between them, every step's image downloaded behind it on the stream, so that a stale or an early
    # row of a neighbouring step would show.
    from vernondsl_b200 import group

    grp = group.Group(dev, world, rank, group.torch_allgather())
    ex = grp.image_exchange(image, W, H, chunk_rows)
    constants = [0.156, 0.21, -0.09]
    hosts = [vd.PinnedArray((H, W), np.uint32) for _ in constants]
    for step, ci in enumerate(constants):
        wire, byte_plane = ex.planes
        for g, p, comb in groups():
            p.ci = ci
            ops.escape_time(st, image, p, wire=wire, byte_plane=byte_plane)
            ex.publish(st, comb)
        ex.complete(st)
        image.download(hosts[step].array, stream=st)
    st.synchronize()
    ex.check()
    for step, ci in enumerate(constants):
        ref, _ = oracle.escape_time(oracle.JULIA, W, H, -1.6, -1.6, dx, dy, -0.8, ci, max_iter)
        if not np.array_equal(hosts[step].array, ref):
            failures.append(f"vrhi_exchange step {step}: {int((hosts[step].array != ref).sum())} pixels differ on rank {rank}")
    # the library's all-reduce: the same bits on every rank, equal to the sum in rank order
    vec = dev.from_numpy((np.arange(5000, dtype=np.float32) * np.float32(0.37) + np.float32(rank) / 8), L.STORAGE_BUFFER)
    for _ in range(2):
        vec.upload((np.arange(5000, dtype=np.float32) * np.float32(0.37) + np.float32(rank) / 8))
        grp.all_reduce_sum(vec, 5000, st)
        st.check()
        expect = np.zeros(5000, np.float32)
        for r in range(world):
            expect = (expect + (np.arange(5000, dtype=np.float32) * np.float32(0.37) + np.float32(r) / 8)).astype(np.float32) if r else (np.arange(5000, dtype=np.float32) * np.float32(0.37) + np.float32(0) / 8)
        if not np.array_equal(vec.download(dtype=np.float32, shape=(5000,)), expect):
            failures.append(f"vrhi_group_all_reduce_sum_f32 differs from the rank-order sum on rank {rank}")
    for h in hosts:
        h.close()
    vec.close()
    dist.barrier()
    ex.close()
    grp.close()
    image.fill(0xEE)
    dev.synchronize()
    dist.barrier()

    # pull form: signals and bounded waits, two wire images alternating
    ex = partition.PullImageExchange(dev, image, plan, W, groups=G, wait_ms=5000)
    for step in range(3):
        for g, p, comb in groups():
            ops.escape_time(st, image, p, wire=ex.wire)
            ex.signal(st, g)
            ex.pull(cst, g, comb)
        torch.cuda.synchronize()
        ex.next_step()
        check(f"pull16 step {step}")
    ex.close()

    dist.barrier()
    dist.destroy_process_group()
    if failures:
        print("\n".join(failures), file=sys.stderr)
        return 1
    if rank == 0:
        print("EXCHANGES_OK")
    return 0


if __name__ == "__main__":
    sys.exit(main())
