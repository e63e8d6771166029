"""GPU: recorded launch sequences and the headless frame loop.

The reference's program re-launches its kernel with a new uniform every frame and blits the field
to a window (fractal.py:28-33).  Here a run of frames is recorded once and replayed with one
submission into a ring of device frames; every frame must equal what a plain launch with that
frame's uniform produces, and the CPU oracle's image, bit for bit."""
import numpy as np
import pytest

import oracle
import vernondsl_b200 as vd
import vernondsl_b200.lang as ti
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu


def _oracle_frame(half, phase):
    ci = float(np.float32(np.cos(np.float32(phase))) * np.float32(0.2))
    d = np.float32(2.0 / half)
    counts, _ = oracle.escape_time(oracle.JULIA, 2 * half, half, -2.0, -1.0, d, d, -0.8, ci, 50,
                                   test=oracle.TEST_NORM_GE, bound=20.0)
    return oracle.escape_color(counts, 0.02).T


def test_frame_loop_replays_a_run_of_frames_into_the_ring():
    ti.init()
    half = 160                      # the reference's own frame: 640 x 320 at n = 320; half of it here
    canvas = ti.field(dtype=float, shape=(half * 2, half))

    @ti.kernel
    def draw(phase: float):
        for a, b in canvas:
            k = ti.Vector([-0.8, ti.cos(phase) * 0.2])
            w = ti.Vector([a / half - 1, b / half - 0.5]) * 2
            steps = 0
            while w.norm() < 20 and steps < 50:
                w = ti.Vector([w[0] ** 2 - w[1] ** 2, w[1] * w[0] * 2]) + k
                steps += 1
            canvas[a, b] = 1 - steps * 0.02

    loop = ti.FrameLoop(draw, canvas, ring=4)
    phases = [k * 0.03 for k in range(6)]
    loop.record(phases)
    st = loop.stream
    before = st.launch_count()
    loop.play()
    assert st.launch_count() - before == 6          # six kernels, one submission
    for k in (2, 3, 4, 5):                          # the ring holds the last four
        assert np.array_equal(loop.frame(k), _oracle_frame(half, phases[k])), k
    with pytest.raises(IndexError):
        loop.frame(1)
    # new uniforms: the recording is re-targeted in place, not rebuilt
    phases2 = [1.0 + k * 0.05 for k in range(6)]
    loop.record(phases2)
    assert loop.seq.stats() == {"kernels": 6, "retargets": 1, "rebuilds": 0}
    loop.play()
    loop.play()                                     # a replay is repeatable
    for k in (2, 5):
        assert np.array_equal(loop.frame(k), _oracle_frame(half, phases2[k])), k
    # a different number of frames changes the shape of the recording: rebuilt, still right
    loop.record(phases[:3])
    assert loop.seq.stats()["rebuilds"] == 1
    loop.play()
    assert np.array_equal(loop.frame(2), _oracle_frame(half, phases[2]))
    # the field itself is untouched as the kernel's target
    draw(0.5)
    assert np.array_equal(canvas.to_numpy(), _oracle_frame(half, 0.5))
    loop.close()


def test_sequence_of_mixed_operators_matches_plain_launches():
    dev = vd.Device(0)
    st = dev.stream()
    rng = np.random.default_rng(11)
    R, Cc = 256, 1024
    a = rng.uniform(-1, 1, R * Cc).astype(np.float32)
    x = rng.standard_normal(R * Cc).astype(np.float32)
    y = rng.standard_normal(R * Cc).astype(np.float32)
    da, dx, dy = (dev.from_numpy(v, L.INPUT) for v in (a, x, y))
    mid = dev.empty((R, Cc), np.float32, L.STORAGE_BUFFER)
    sums = dev.empty((R,), np.float32, L.OUTPUT)
    cols = dev.empty((Cc,), np.float32, L.OUTPUT)
    soft = dev.empty((R, Cc), np.float32, L.OUTPUT)

    def chain():
        ops.fused_map(st, da, dx, dy, mid, R * Cc)
        ops.row_sum(st, mid, sums, R, Cc)
        ops.col_sum(st, mid, cols, R, Cc)
        ops.row_softmax(st, mid, soft, R, Cc)

    chain()                                         # plain launches (also sizes the stream scratch)
    st.check()
    want = [b.download(dtype=np.float32) for b in (mid, sums, cols, soft)]
    for b in (mid, sums, cols, soft):
        b.fill(0, stream=st)
    with st.record() as seq:
        chain()
    st.check()
    assert not np.any(sums.download(dtype=np.float32)), "recording must not execute"
    assert seq.stats()["kernels"] >= 4
    seq.launch()
    st.check()
    got = [b.download(dtype=np.float32) for b in (mid, sums, cols, soft)]
    for g, w in zip(got, want):
        assert np.array_equal(g, w)                 # same kernels, same order of operations: same bits
    seq.close()
    st.close()


def test_recording_refuses_an_operator_whose_scratch_does_not_exist_yet():
    dev = vd.Device(0)
    st = dev.stream()                               # fresh stream: no scratch yet
    img = dev.empty((64, 64), np.uint32, L.IMAGE)
    p = ops.escape_params(L.MANDELBROT, 64, 64, -2.5, -1.0, 3.5 / 64, 2.0 / 64, max_iter=128)
    with pytest.raises(vd.VrhiError) as err:
        with st.record():
            ops.escape_time(st, img, p)
    assert err.value.status == L.ERR_INVALID and "before recording" in str(err.value)
    ops.escape_time(st, img, p)                     # the stream is usable afterwards
    st.check()
    want, _ = oracle.escape_time(oracle.MANDELBROT, 64, 64, -2.5, -1.0, np.float32(3.5 / 64), np.float32(2.0 / 64), max_iter=128)
    assert np.array_equal(img.download(dtype=np.uint32, shape=(64, 64)), want)
    st.close()


def test_a_recording_can_span_two_streams():
    """Frames of a loop go to two streams in turn inside one recording; every frame must still be right,
    and launching on a side stream that was not drawn into the recording must fail loudly."""
    dev = vd.Device(0)
    st, side, stray = dev.stream(), dev.stream(), dev.stream()
    W, H, N = 640, 360, 200
    dx, dy = ops.grid_steps(-2.5, 1.0, -1.0, 1.0, W, H)
    want, _ = oracle.escape_time(oracle.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=N)
    ring = [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(4)]
    p = ops.escape_params(L.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=N)
    for s in (st, side):
        ops.escape_time(s, ring[0], p)       # sizes each stream's scratch
        s.check()
    for b in ring:
        b.fill(0, stream=st)
    st.check()
    with st.record() as seq:
        st.fork_recording(side)
        with pytest.raises(vd.VrhiError):
            st.fork_recording(side)           # already part of the recording
        for k in range(8):
            ops.escape_time(st if k % 2 == 0 else side, ring[k % 4], p)
    assert seq.stats()["kernels"] == 8
    assert not np.any(ring[1].download(dtype=np.uint32, shape=(H, W))), "recording must not execute"
    before = st.launch_count(), side.launch_count()
    seq.launch()
    st.check()
    assert (st.launch_count() - before[0], side.launch_count() - before[1]) == (8, 0)
    for b in ring:
        assert np.array_equal(b.download(dtype=np.uint32, shape=(H, W)), want)
    with pytest.raises(vd.VrhiError):
        stray.fork_recording(side)            # `stray` is not recording
    seq.close()
    for s in (st, side, stray):
        s.close()


def test_a_sequence_survives_the_growth_of_its_streams_scratch(dev, stream):
    """A recorded sequence points into the stream's scratch of its time (the escape-time work counter
    and the memset that clears it).  An operator that later needs more scratch than the stream holds
    makes the stream allocate a larger block; the block the sequence points into must stay alive,
    and both the sequence and the operator must keep giving right answers."""
    W = H = 512
    dx, dy = ops.grid_steps(-1.6, 1.6, -1.6, 1.6, W, H)
    p = ops.escape_params(L.JULIA, W, H, -1.6, -1.6, dx, dy, cr=-0.8, ci=0.156, max_iter=300)
    img = dev.empty((H, W), np.uint32, L.IMAGE)
    ops.escape_time(stream, img, p)          # sizes the scratch (4 MiB at first use)
    stream.check()
    with stream.record() as seq:
        ops.escape_time(stream, img, p)
    want, _ = oracle.escape_time(oracle.JULIA, W, H, -1.6, -1.6, dx, dy, -0.8, 0.156, 300)
    # column sums of [4096, 8192]: the partial rows need well over 4 MiB of scratch
    rows, cols = 4096, 8192
    m = np.random.default_rng(3).standard_normal((rows, cols)).astype(np.float32)
    M, out = dev.from_numpy(m), dev.empty(cols, np.float32)
    for _ in range(2):
        img.fill(0)
        seq.launch()
        ops.col_sum(stream, M, out, rows, cols)
        seq.launch()
        stream.check()
        assert np.array_equal(img.download(), want)
        got = out.download()
        ref = m.astype(np.float64).sum(axis=0)
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(m).astype(np.float64).sum(axis=0).max()
    seq.close()
    for b in (img, M, out):
        b.close()


# --------------------------------------------------------------------------------------------------
# Launches declared independent of their predecessors (VRHI_ESCAPE_INDEPENDENT_OF): frames that go
# round a ring on ONE stream and may begin before the frames before them end.  Every frame must
# still be, bit for bit, what an ordered launch with the same parameters writes.

def _view_params(k, W, H, independent_of, max_iter=256):
    dx, dy = ops.grid_steps(-2.5 + 0.01 * k, 1.0 + 0.01 * k, -1.0, 1.0, W, H)
    return ops.escape_params(L.MANDELBROT, W, H, -2.5 + 0.01 * k, -1.0, dx, dy, max_iter=max_iter, independent_of=independent_of)


@pytest.mark.parametrize("recorded", [False, True])
@pytest.mark.parametrize("ring_size,independent_of", [(4, 3), (2, 1), (8, 7)])
def test_independent_launches_on_one_stream_write_the_frames_ordered_launches_write(dev, stream, recorded, ring_size, independent_of):
    W, H, frames = 960, 544, 2 * ring_size + 3          # work-stealing kernel, two pixels per lane
    want = []
    scratch = dev.empty((H, W), np.uint32, L.IMAGE)
    for k in range(frames):
        ops.escape_time(stream, scratch, _view_params(k, W, H, 0))
        stream.check()
        want.append(scratch.download(dtype=np.uint32, shape=(H, W)))
    counts, _ = oracle.escape_time(oracle.MANDELBROT, W, H, -2.5 + 0.01 * (frames - 1), -1.0,
                                   *ops.grid_steps(-2.5 + 0.01 * (frames - 1), 1.0 + 0.01 * (frames - 1), -1.0, 1.0, W, H), 0.0, 0.0, 256)
    assert np.array_equal(want[-1], counts)
    ring = [dev.empty((H, W), np.uint32, L.IMAGE) for _ in range(ring_size)]

    def run():
        for k in range(frames):
            ops.escape_time(stream, ring[k % ring_size], _view_params(k, W, H, independent_of))

    def check():
        stream.check()
        for k in range(frames - ring_size, frames):
            assert np.array_equal(ring[k % ring_size].download(dtype=np.uint32, shape=(H, W)), want[k]), k

    if not recorded:
        for _ in range(3):
            for b in ring:
                b.fill(0xEE, stream=stream)
            before = stream.launch_count()
            run()
            assert stream.launch_count() - before == frames
            check()
    else:
        with stream.record() as seq:
            run()
        assert seq.stats()["kernels"] == frames
        for _ in range(3):
            for b in ring:
                b.fill(0xEE, stream=stream)
            seq.launch(stream)
            check()
        seq.launch(stream)          # replays back to back: the second begins behind the whole of the first
        seq.launch(stream)
        check()
        seq.close()
    # an ordered launch right behind a run sees the run finished: it overwrites the last frame's slot
    run()
    last = (frames - 1) % ring_size
    ops.escape_time(stream, ring[last], _view_params(0, W, H, 0))
    stream.check()
    assert np.array_equal(ring[last].download(dtype=np.uint32, shape=(H, W)), want[0])
    for b in ring + [scratch]:
        b.close()


def test_independent_small_frames_dealt_without_a_counter(dev, stream):
    """The reference's own frame (fractal.py:7-25, 640 x 320 colour, at most 50 steps) runs the kernel that deals
    its batches statically; a run of such frames, each with its own uniform, overlaps on one stream."""
    half, frames = 320, 16
    d = float(np.float32(2.0 / half))
    phases = [0.03 * k for k in range(frames)]
    ring = [dev.empty((2 * half, half), np.float32, L.IMAGE) for _ in range(4)]

    def params(phase, k):
        return ops.escape_params(L.JULIA, half, 2 * half, -1.0, -2.0, d, d, cr=-0.8, transposed=True,
                                 ci=float(np.float32(np.cos(np.float32(phase))) * np.float32(0.2)), max_iter=50,
                                 test=L.TEST_NORM_GE, bound=20.0, output=L.OUT_COLOR_F32, color_scale=0.02, independent_of=k)

    for k, ph in enumerate(phases):
        ops.escape_time(stream, ring[k % 4], params(ph, 3))
    stream.check()
    for k in range(frames - 4, frames):
        assert np.array_equal(ring[k % 4].download(dtype=np.float32, shape=(2 * half, half)), _oracle_frame(half, phases[k])), k
    # a run broken by a launch that declares nothing, and by one that declares less than the run is long
    for k, ph in enumerate(phases):
        ops.escape_time(stream, ring[k % 4], params(ph, (3, 3, 0, 1, 3, 2)[k % 6]))
    stream.check()
    for k in range(frames - 4, frames):
        assert np.array_equal(ring[k % 4].download(dtype=np.float32, shape=(2 * half, half)), _oracle_frame(half, phases[k])), k
    for b in ring:
        b.close()


def test_frame_loop_on_one_stream_overlaps_its_frames():
    ti.init()
    half = 160
    canvas = ti.field(dtype=float, shape=(half * 2, half))

    @ti.kernel
    def draw(phase: float):
        for a, b in canvas:
            k = ti.Vector([-0.8, ti.cos(phase) * 0.2])
            w = ti.Vector([a / half - 1, b / half - 0.5]) * 2
            steps = 0
            while w.norm() < 20 and steps < 50:
                w = ti.Vector([w[0] ** 2 - w[1] ** 2, w[1] * w[0] * 2]) + k
                steps += 1
            canvas[a, b] = 1 - steps * 0.02

    loop = ti.FrameLoop(draw, canvas, ring=4, streams=1)
    assert loop.independent_of == 3 and len(loop.streams) == 1
    phases = [k * 0.03 for k in range(9)]
    loop.record(phases)
    assert (draw.last_params.flags >> 8) & 7 == 3
    loop.play()
    loop.play()
    for k in (5, 6, 7, 8):
        assert np.array_equal(loop.frame(k), _oracle_frame(half, phases[k])), k
    draw(0.5)                                        # outside the loop the kernel declares nothing
    assert (draw.last_params.flags >> 8) & 7 == 0
    assert np.array_equal(canvas.to_numpy(), _oracle_frame(half, 0.5))
    loop.close()
