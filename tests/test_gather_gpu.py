"""GPU: the uint16 wire copy of the escape-time counts and the widening kernel of the image gather.

The two ranks of a world are played one after the other on one GPU (each computes its own chunks into
its own image and wire image), the peer push is a strided device copy between the wire images, and
the widened result must equal the CPU oracle's whole image bit for bit."""
import numpy as np
import pytest

import oracle
import vernondsl_b200 as vd
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu

J = dict(x0=-1.6, y0=-1.6, cr=-0.8, ci=0.156)


def _julia(W, H, max_iter):
    dx, dy = ops.grid_steps(-1.6, 1.6, -1.6, 1.6, W, H)
    want, _ = oracle.escape_time(oracle.JULIA, W, H, J["x0"], J["y0"], dx, dy, J["cr"], J["ci"], max_iter)
    return dx, dy, want


@pytest.mark.parametrize("max_iter,checked", [(300, False), (300, True), (40, False)])
def test_wire_copy_equals_the_counts(max_iter, checked):
    dev = vd.Device(0)
    st = dev.stream()
    W, H = 520, 96                      # width not a multiple of 32: ragged last tile
    dx, dy, want = _julia(W, H, max_iter)
    img = dev.empty((H, W), np.uint32, L.IMAGE)
    wire = dev.empty((H, W), np.uint16, L.IMAGE)
    p = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=max_iter, checked_only=checked)
    ops.escape_time(st, img, p, wire=wire)
    st.check()
    assert np.array_equal(img.download(dtype=np.uint32, shape=(H, W)), want)
    assert np.array_equal(wire.download(dtype=np.uint16, shape=(H, W)), want.astype(np.uint16))
    st.close()


def test_wire_copy_is_refused_where_it_would_lose_counts():
    dev = vd.Device(0)
    st = dev.stream()
    img = dev.empty((32, 64), np.uint32, L.IMAGE)
    wire = dev.empty((32, 64), np.uint16, L.IMAGE)
    p = ops.escape_params(L.MANDELBROT, 64, 32, -2.5, -1.0, 3.5 / 64, 2.0 / 32, max_iter=70000)
    with pytest.raises(vd.VrhiError) as err:
        ops.escape_time(st, img, p, wire=wire)
    assert err.value.status == L.ERR_UNSUPPORTED
    small = dev.empty((16, 64), np.uint16, L.IMAGE)
    p.max_iter = 100
    with pytest.raises(vd.VrhiError) as err:
        ops.escape_time(st, img, p, wire=small)
    assert err.value.status == L.ERR_SIZE
    st.close()


@pytest.mark.parametrize("W,world", [(512, 2), (512, 4), (100, 2)])   # 100: the scalar path of the widening kernel
def test_gather_with_uint16_on_the_wire_rebuilds_the_whole_image(W, world):
    dev = vd.Device(0)
    st = dev.stream()
    chunk_rows, slabs = 8, 3
    H = chunk_rows * world * slabs
    max_iter = 400
    dx, dy, want = _julia(W, H, max_iter)
    images = [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(world)]
    wires = [dev.empty((H, W), np.uint16, L.IMAGE) for _ in range(world)]
    for r in range(world):
        images[r].fill(0xEE, stream=st)           # rows of other ranks start as garbage
        wires[r].fill(0xDD, stream=st)
        part = ops.partition_rows(H, world, r, L.PART_CYCLIC, chunk_rows)
        p = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=max_iter, partition=part)
        ops.escape_time(st, images[r], p, wire=wires[r])
    # the push: rank r's chunks (every world-th chunk starting at r) into every peer's wire image
    chunk_bytes = chunk_rows * W * 2
    for r in range(world):
        for q in range(world):
            if q != r:
                wires[r].copy_2d_to(wires[q], r * chunk_bytes, world * chunk_bytes, r * chunk_bytes, world * chunk_bytes, chunk_bytes, slabs, st)
    # arrival, in two combs of slabs as a pipelined step does it: slabs 0 and 2, then slab 1
    for r in range(world):
        ops.widen_rows_u16(st, wires[r], images[r], W, H, chunk_rows, world, r, 0, 2, 2)
        ops.widen_rows_u16(st, wires[r], images[r], W, H, chunk_rows, world, r, 1, 1, 2)
    st.check()
    for r in range(world):
        assert np.array_equal(images[r].download(dtype=np.uint32, shape=(H, W)), want), r
    # widening every chunk (no rank skipped) from a complete wire image gives the same picture
    blank = dev.empty((H, W), np.uint32, L.IMAGE)
    blank.fill(0, stream=st)
    ops.widen_rows_u16(st, wires[0], blank, W, H, chunk_rows, world, world, 0, slabs)
    st.check()
    assert np.array_equal(blank.download(dtype=np.uint32, shape=(H, W)), want)
    with pytest.raises(vd.VrhiError):
        ops.widen_rows_u16(st, wires[0], blank, W, H, chunk_rows, world, 0, slabs, 1)   # beyond the last slab
    st.close()


@pytest.mark.parametrize("world,max_iter", [(2, 400), (4, 400), (4, 200)])
def test_gather_with_a_byte_plane_rebuilds_the_whole_image(world, max_iter):
    """The squeezed form of the gather, ranks played one after the other on one GPU: the kernel writes
    min(count, 255) into a byte plane beside the uint16 wire image, only the byte plane is pushed,
    and the widening kernel fetches the granules that show a byte of 255 from the owner's wire image
    (here: another buffer on the same GPU).  max_iter 200 leaves no count above 254: nothing is fetched."""
    dev = vd.Device(0)
    st = dev.stream()
    W, chunk_rows, slabs = 512, 8, 3
    H = chunk_rows * world * slabs
    dx, dy, want = _julia(W, H, max_iter)
    assert (want >= 255).any() == (max_iter > 254)
    images = [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(world)]
    wires = [dev.empty((H, W), np.uint16, L.IMAGE) for _ in range(world)]
    planes = [dev.empty((H, W), np.uint8, L.IMAGE) for _ in range(world)]
    for r in range(world):
        images[r].fill(0xEE, stream=st)
        wires[r].fill(0xDD, stream=st)
        planes[r].fill(0xCC, stream=st)
        part = ops.partition_rows(H, world, r, L.PART_CYCLIC, chunk_rows)
        p = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=max_iter, partition=part)
        ops.escape_time(st, images[r], p, wire=wires[r], byte_plane=planes[r])
    st.check()
    # the byte plane of a rank holds min(count, 255) on the rank's own rows
    own0 = np.zeros(H, bool)
    for k in range(slabs):
        own0[(k * world) * chunk_rows:(k * world + 1) * chunk_rows] = True
    got = planes[0].download(dtype=np.uint8, shape=(H, W))
    assert np.array_equal(got[own0], np.minimum(want[own0], 255).astype(np.uint8))
    # the push: rank r's chunks of the BYTE plane into every peer's byte plane; the wire images stay where they are
    chunk_bytes = chunk_rows * W
    for r in range(world):
        for q in range(world):
            if q != r:
                planes[r].copy_2d_to(planes[q], r * chunk_bytes, world * chunk_bytes, r * chunk_bytes, world * chunk_bytes, chunk_bytes, slabs, st)
    for r in range(world):
        ops.widen_rows_u8(st, planes[r], images[r], wires, W, H, chunk_rows, world, r, 0, 2, 2)
        ops.widen_rows_u8(st, planes[r], images[r], wires, W, H, chunk_rows, world, r, 1, 1, 2)
    st.check()
    for r in range(world):
        assert np.array_equal(images[r].download(dtype=np.uint32, shape=(H, W)), want), r
    st.close()


def test_pull_gather_reads_the_peers_rows_and_widens_them():
    dev = vd.Device(0)
    st = dev.stream()
    W, world, chunk_rows, slabs = 256, 3, 4, 5
    H = chunk_rows * world * slabs
    max_iter = 500
    dx, dy, want = _julia(W, H, max_iter)
    images = [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(world)]
    wires = [dev.empty((H, W), np.uint16, L.IMAGE) for _ in range(world)]
    flags = [dev.empty((world,), np.uint32, L.STORAGE_BUFFER) for _ in range(world)]
    for r in range(world):
        images[r].fill(0xEE, stream=st)
        wires[r].fill(0xDD, stream=st)
        flags[r].fill(0, stream=st)
        part = ops.partition_rows(H, world, r, L.PART_CYCLIC, chunk_rows)
        p = ops.escape_params(L.JULIA, W, H, J["x0"], J["y0"], dx, dy, cr=J["cr"], ci=J["ci"], max_iter=max_iter, partition=part)
        ops.escape_time(st, images[r], p, wire=wires[r])
    seq = 7
    for r in range(world):          # every rank marks its rows ready in its peers' flag arrays
        ops.gather_signal(st, [flags[q] for q in range(world) if q != r], world, r, seq)
    for r in range(world):          # the marks are already there (same stream): the wait returns at once
        peers = [wires[q] for q in range(world) if q != r]
        ops.gather_pull_u16(st, flags[r], images[r], peers, W, H, chunk_rows, world, r, 0, 3, seq, wait_ms=200, slab_stride=2)   # slabs 0, 2, 4
        ops.gather_pull_u16(st, flags[r], images[r], peers, W, H, chunk_rows, world, r, 1, 2, seq - 3, wait_ms=200, slab_stride=2)  # slabs 1, 3; an older number is satisfied too
    st.check()
    for r in range(world):
        got_flags = flags[r].download(dtype=np.uint32)
        assert [int(v) for v in got_flags] == [0 if q == r else seq for q in range(world)]
        assert np.array_equal(images[r].download(dtype=np.uint32, shape=(H, W)), want), r
    st.close()


def test_pull_gather_gives_up_after_its_time_limit_and_reports_it():
    """A flag that nothing sets: the device-side wait runs out, the kernel copies nothing and returns,
    the stream reports VRHI_ERR_TIMEOUT once and stays usable."""
    dev = vd.Device(0)
    st = dev.stream()
    W, H, world, chunk_rows = 64, 16, 2, 4
    image = dev.empty((H, W), np.uint32, L.IMAGE)
    wire_peer = dev.empty((H, W), np.uint16, L.IMAGE)
    flags = dev.empty((world,), np.uint32, L.STORAGE_BUFFER)
    image.fill(0x11, stream=st)
    wire_peer.fill(0x22, stream=st)
    flags.fill(0, stream=st)
    ops.gather_pull_u16(st, flags, image, [wire_peer], W, H, chunk_rows, world, 0, 0, 2, seq=1, wait_ms=20)
    with pytest.raises(vd.VrhiError) as err:
        st.check()
    assert err.value.status == L.ERR_TIMEOUT
    assert np.all(image.download(dtype=np.uint32, shape=(H, W)) == 0x11111111)      # untouched
    st.check()                                                                       # reported once; the stream goes on
    ops.gather_signal(st, [flags], world, 1, 1)                                      # the peer's mark arrives
    ops.gather_pull_u16(st, flags, image, [wire_peer], W, H, chunk_rows, world, 0, 0, 2, seq=1, wait_ms=20)
    st.check()
    got = image.download(dtype=np.uint32, shape=(H, W))
    rows_of_peer = [r for r in range(H) if (r // chunk_rows) % world == 1]
    rows_own = [r for r in range(H) if (r // chunk_rows) % world == 0]
    assert np.all(got[rows_of_peer] == 0x2222) and np.all(got[rows_own] == 0x11111111)
    st.close()
