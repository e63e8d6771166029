"""GPU: escape-time kernels against the CPU oracle, bit for bit, through the C ABI."""
import numpy as np
import pytest

import oracle
from tests.golden.make_golden import WORKLOADS
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu


def run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, dtype=np.uint32, **kw):
    out = dev.empty((H, W), dtype, L.IMAGE)
    out.fill(0xCD)
    p = ops.escape_params(kind, W, H, x0, y0, dx, dy, **kw)
    ops.escape_time(stream, out, p)
    stream.check()
    img = out.download()
    out.close()
    return img


def workload(name):
    kind, W, H, x0, x1, y0, y1, cr, ci, mi = WORKLOADS[name]
    dx, dy = oracle.grid_steps(x0, x1, y0, y1, W, H)
    return kind, W, H, np.float32(x0), np.float32(y0), dx, dy, dict(cr=cr, ci=ci, max_iter=mi)


@pytest.mark.parametrize("name", ["mandelbrot_1080p", "julia_512", "mandelbrot_ragged"])
def test_counts_equal_oracle(dev, stream, name):
    kind, W, H, x0, y0, dx, dy, kw = workload(name)
    got = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, **kw)
    want, total = oracle.escape_time(kind, W, H, x0, y0, dx, dy, kw["cr"], kw["ci"], kw["max_iter"])
    assert np.array_equal(got, want)
    assert int(got.sum(dtype=np.uint64)) == total


@pytest.mark.parametrize("name", ["mandelbrot_1080p", "julia_512", "mandelbrot_ragged"])
def test_step_by_step_kernel_equals_oracle_too(dev, stream, name):
    """The same workloads forced onto the kernel that tests on every step."""
    kind, W, H, x0, y0, dx, dy, kw = workload(name)
    got = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, checked_only=True, **kw)
    want, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, kw["cr"], kw["ci"], kw["max_iter"])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("max_iter", [2, 7, 8, 9, 15, 16, 17, 100])
def test_max_iter_around_the_block_length(dev, stream, max_iter):
    """Counts that stop at max_iter inside, at the edge of and just past an unchecked block."""
    dx, dy = oracle.grid_steps(-1.6, 1.6, -1.6, 1.6, 260, 96)
    for kind, cr, ci in ((L.JULIA, -0.8, 0.156), (L.JULIA, 0.0, 0.0), (L.MANDELBROT, 0.0, 0.0)):
        got = run_gpu(dev, stream, kind, 260, 96, -1.6, -1.6, dx, dy, cr=cr, ci=ci, max_iter=max_iter)
        want, _ = oracle.escape_time(kind, 260, 96, -1.6, -1.6, dx, dy, cr, ci, max_iter)
        assert np.array_equal(got, want)


def test_interior_heavy_image(dev, stream):
    """Nearly every pixel runs to max_iter (a zoom into the set): the pool stays full throughout."""
    dx, dy = oracle.grid_steps(-0.2, 0.2, -0.2, 0.2, 384, 128)
    got = run_gpu(dev, stream, L.MANDELBROT, 384, 128, -0.2, -0.2, dx, dy, max_iter=1000)
    want, _ = oracle.escape_time(oracle.MANDELBROT, 384, 128, -0.2, -0.2, dx, dy, max_iter=1000)
    assert np.array_equal(got, want) and (want == 1000).mean() > 0.9


def test_full_size_julia_equals_golden_digest(dev, stream, golden):
    """16384 x 16384, max_iter 4096: compared through the exact digests the oracle produced, and
    row by row on the stored sample rows."""
    kind, W, H, x0, y0, dx, dy, kw = workload("julia_16k")
    got = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, **kw)
    s, w = oracle.digest_u32(got)
    assert [s, w] == [int(v) for v in golden["julia_16k_digest"]]
    rows = golden["julia_16k_rows"]
    assert np.array_equal(got[rows], golden["julia_16k_row_counts"].astype(np.uint32))
    # live oracle on a band of rows through the dense part of the set
    band = np.arange(8000, 8000 + 64)
    want, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, kw["cr"], kw["ci"], kw["max_iter"], row_begin=8000, row_step=1, row_count=64)
    assert np.array_equal(got[band], want)


@pytest.mark.parametrize("W,H", [(1, 1), (1, 7), (31, 3), (33, 2), (513, 5), (4097, 3)])
def test_ragged_shapes(dev, stream, W, H):
    dx, dy = oracle.grid_steps(-2.0, 1.0, -1.2, 1.2, W, H)
    got = run_gpu(dev, stream, L.MANDELBROT, W, H, -2.0, -1.2, dx, dy, max_iter=200)
    want, _ = oracle.escape_time(oracle.MANDELBROT, W, H, -2.0, -1.2, dx, dy, max_iter=200)
    assert np.array_equal(got, want)


def test_max_iter_zero_and_one(dev, stream):
    for mi in (0, 1):
        dx, dy = oracle.grid_steps(-2.0, 1.0, -1.2, 1.2, 64, 8)
        got = run_gpu(dev, stream, L.MANDELBROT, 64, 8, -2.0, -1.2, dx, dy, max_iter=mi)
        want, _ = oracle.escape_time(oracle.MANDELBROT, 64, 8, -2.0, -1.2, dx, dy, max_iter=mi)
        assert np.array_equal(got, want)


def test_julia_with_large_constant_takes_the_checked_path(dev, stream):
    # |c| > 1.5: escape is not guaranteed monotonic, so only the step-by-step kernel may run it
    dx, dy = oracle.grid_steps(-2.0, 2.0, -2.0, 2.0, 200, 120)
    for cr, ci in [(-1.9, 0.1), (1.6, 1.2), (-2.2, 0.0)]:
        got = run_gpu(dev, stream, L.JULIA, 200, 120, -2.0, -2.0, dx, dy, cr=cr, ci=ci, max_iter=500)
        want, _ = oracle.escape_time(oracle.JULIA, 200, 120, -2.0, -2.0, dx, dy, cr, ci, 500)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("bound", [4.0, 16.0, 2.0, 0.5])
def test_other_bounds(dev, stream, bound):
    dx, dy = oracle.grid_steps(-1.6, 1.6, -1.6, 1.6, 300, 100)
    got = run_gpu(dev, stream, L.JULIA, 300, 100, -1.6, -1.6, dx, dy, cr=-0.8, ci=0.156, max_iter=700, bound=bound)
    want, _ = oracle.escape_time(oracle.JULIA, 300, 100, -1.6, -1.6, dx, dy, -0.8, 0.156, 700, bound=bound)
    assert np.array_equal(got, want)


def test_fractal_py_paint_semantics(dev, stream):
    """fractal.py:16-25: 640 x 320 field, z = ((i/n - 1)*2, (j/n - 0.5)*2), c = (-0.8, cos(t)*0.2),
    `while z.norm() < 20 and iterations < 50`, pixel = 1 - iterations*0.02."""
    n = 320
    W, H = 2 * n, n  # the field is indexed [i, j] with i the long axis; rows of the image are j
    d = np.float32(2.0 / n)
    for t in (0.0, 0.9):
        ci = float(np.float32(np.cos(np.float32(t))) * np.float32(0.2))
        counts = run_gpu(dev, stream, L.JULIA, W, H, -2.0, -1.0, d, d, cr=-0.8, ci=ci, max_iter=50,
                         test=L.TEST_NORM_GE, bound=20.0)
        want, _ = oracle.escape_time(oracle.JULIA, W, H, -2.0, -1.0, d, d, -0.8, ci, 50, test=oracle.TEST_NORM_GE, bound=20.0)
        assert np.array_equal(counts, want)
        colour = run_gpu(dev, stream, L.JULIA, W, H, -2.0, -1.0, d, d, dtype=np.float32, cr=-0.8, ci=ci, max_iter=50,
                         test=L.TEST_NORM_GE, bound=20.0, output=L.OUT_COLOR_F32, color_scale=0.02)
        assert np.array_equal(colour, oracle.escape_color(want, 0.02))


def test_uint16_output(dev, stream):
    kind, W, H, x0, y0, dx, dy, kw = workload("julia_512")
    got = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, dtype=np.uint16, output=L.OUT_COUNT_U16, **kw)
    want, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, kw["cr"], kw["ci"], kw["max_iter"])
    assert np.array_equal(got.astype(np.uint32), want)
    with pytest.raises(L.VrhiError) as e:
        run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, dtype=np.uint16, output=L.OUT_COUNT_U16, cr=0.0, ci=0.0, max_iter=70000)
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("scheme,chunk,world", [(L.PART_CYCLIC, 16, 4), (L.PART_CYCLIC, 128, 8), (L.PART_CONTIGUOUS, 0, 4), (L.PART_CYCLIC, 7, 3)])
def test_row_partitions_tile_the_image(dev, stream, scheme, chunk, world):
    """Every rank's launch writes only its own rows, at their true place; together they give the image."""
    kind, W, H, x0, y0, dx, dy, kw = workload("julia_512")
    H = 500  # not a multiple of the chunk sizes
    want, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, kw["cr"], kw["ci"], kw["max_iter"])
    out = dev.empty((H, W), np.uint32, L.IMAGE)
    out.fill(0xFF)
    owners = np.full(H, -1)
    for rank in range(world):
        part = ops.partition_rows(H, world, rank, scheme, chunk)
        before = out.download()
        ops.escape_time(stream, out, ops.escape_params(kind, W, H, x0, y0, dx, dy, partition=part, **kw))
        stream.check()
        after = out.download()
        changed = np.where((before != after).any(axis=1))[0]
        assert (owners[changed] == -1).all()
        owners[changed] = rank
        assert len(changed) == part.rows_owned
    assert (owners >= 0).all()
    assert np.array_equal(out.download(), want)
    out.close()


def test_fast_mode_is_close_but_reported_separately(dev, stream):
    kind, W, H, x0, y0, dx, dy, kw = workload("julia_512")
    exact = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, **kw)
    fast = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, mode=L.FAST, **kw)
    # the contracted mode is itself a fixed rounding sequence: both kernels reproduce the oracle's bits
    want_fast, _ = oracle.escape_time(kind, W, H, x0, y0, dx, dy, kw["cr"], kw["ci"], kw["max_iter"], fast=True)
    assert np.array_equal(fast, want_fast)
    fast_checked = run_gpu(dev, stream, kind, W, H, x0, y0, dx, dy, mode=L.FAST, checked_only=True, **kw)
    assert np.array_equal(fast_checked, want_fast)
    mkind, mW, mH, mx0, my0, mdx, mdy, mkw = workload("mandelbrot_ragged")
    mfast = run_gpu(dev, stream, mkind, mW, mH, mx0, my0, mdx, mdy, mode=L.FAST, **mkw)
    mwant, _ = oracle.escape_time(mkind, mW, mH, mx0, my0, mdx, mdy, max_iter=mkw["max_iter"], fast=True)
    assert np.array_equal(mfast, mwant)
    mismatch = float((exact != fast).mean())
    assert mismatch < 0.05  # contraction changes roundings: some boundary pixels move
    assert abs(int(fast.sum(dtype=np.int64)) - int(exact.sum(dtype=np.int64))) < 0.02 * exact.sum(dtype=np.int64)


def test_argument_errors(dev, stream):
    img = dev.empty((8, 8), np.uint32, L.IMAGE)
    ro = dev.empty((8, 8), np.uint32, L.INPUT)
    p = ops.escape_params(L.JULIA, 8, 8, 0, 0, 0.1, 0.1)
    with pytest.raises(L.VrhiError) as e:
        ops.launch(stream, "escape_time", [ro.arg(L.OUTPUT)], p)
    assert e.value.status == L.ERR_INVALID and "read-only" in e.value.message
    big = ops.escape_params(L.JULIA, 64, 64, 0, 0, 0.1, 0.1)
    with pytest.raises(L.VrhiError) as e:
        ops.escape_time(stream, img, big)
    assert e.value.status == L.ERR_SIZE
    bad = ops.escape_params(7, 8, 8, 0, 0, 0.1, 0.1)
    with pytest.raises(L.VrhiError) as e:
        ops.escape_time(stream, img, bad)
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.VrhiError) as e:
        ops.launch(stream, "escape_time", [img.arg(L.OUTPUT, offset=8)], p)
    assert e.value.status == L.ERR_SIZE
    img.close()
    ro.close()
