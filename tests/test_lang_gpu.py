"""GPU: the Taichi-style front end.  A program written the way the reference's fractal.py is written
(struct-for over a field, a @func for the complex square, a while loop on the norm, a colour
store) must run as ONE escape_time launch and agree with the CPU oracle bit for bit; elementwise
bodies must become ONE fused map kernel."""
import numpy as np
import pytest

import oracle
import vernondsl_b200.lang as ti
from vernondsl_b200 import _lib as L

pytestmark = pytest.mark.gpu


def test_julia_program_in_the_style_of_fractal_py():
    ti.init(arch=ti.gles)   # the reference asks for an OpenGL ES device; here it is the CUDA device
    half = 96
    shade = ti.field(dtype=float, shape=(half * 2, half))

    @ti.func
    def csq(w):
        return ti.Vector([w[0] ** 2 - w[1] ** 2, w[1] * w[0] * 2])

    @ti.kernel
    def draw(phase: float):
        for a, b in shade:
            k = ti.Vector([-0.8, ti.cos(phase) * 0.2])
            w = ti.Vector([a / half - 1, b / half - 0.5]) * 2
            steps = 0
            while w.norm() < 20 and steps < 50:
                w = csq(w) + k
                steps += 1
            shade[a, b] = 1 - steps * 0.02

    for frame in range(3):           # the frame loop: a new uniform, a relaunch
        phase = frame * 0.03
        draw(phase)
        got = shade.to_numpy()
        assert "escape_time" in draw.last_plan and "transposed=True" in draw.last_plan
        # oracle: real axis = first field index (rows here), imaginary = second index (columns)
        ci = float(np.float32(np.cos(np.float32(phase))) * np.float32(0.2))
        d = np.float32(2.0 / half)
        counts, _ = oracle.escape_time(oracle.JULIA, 2 * half, half, -2.0, -1.0, d, d, -0.8, ci, 50,
                                       test=oracle.TEST_NORM_GE, bound=20.0)
        want = oracle.escape_color(counts, 0.02).T     # oracle image is [imag][real]; the field is [real][imag]
        assert got.shape == (2 * half, half)
        assert np.array_equal(got, want)
    assert got.min() >= 0.0 and got.max() <= 1.0 and len(np.unique(got)) > 10


def test_mandelbrot_counts_into_an_integer_field():
    ti.init()
    W, H, N = 200, 120, 300
    img = ti.field(dtype=int, shape=(H, W))

    @ti.kernel
    def mandel():
        for r, c in img:
            k = ti.Vector([c * (3.5 / W) - 2.5, r * (2.0 / H) - 1.0])
            z = ti.Vector([0.0, 0.0])
            n = 0
            while z.norm_sqr() <= 4 and n < N:
                z = ti.Vector([z[0] * z[0] - z[1] * z[1], 2 * z[0] * z[1]]) + k
                n += 1
            img[r, c] = n

    mandel()
    assert "mandelbrot" in mandel.last_plan and "transposed=False" in mandel.last_plan
    dx, dy = np.float32(3.5 / W), np.float32(2.0 / H)
    want, _ = oracle.escape_time(oracle.MANDELBROT, W, H, -2.5, -1.0, dx, dy, max_iter=N)
    assert np.array_equal(img.to_numpy().astype(np.uint32), want)


def test_elementwise_body_becomes_one_fused_kernel():
    ti.init()
    R, Cc = 48, 256
    rng = np.random.default_rng(5)
    a, x, y, out, out2 = (ti.field(float, (R, Cc)) for _ in range(5))
    bias = ti.field(float, (Cc,))
    av, xv, yv = rng.uniform(-1, 1, (R, Cc)).astype(np.float32), rng.standard_normal((R, Cc)).astype(np.float32), rng.standard_normal((R, Cc)).astype(np.float32)
    bv = rng.standard_normal(Cc).astype(np.float32)
    a.from_numpy(av); x.from_numpy(xv); y.from_numpy(yv); bias.from_numpy(bv)

    @ti.kernel
    def chain(gain: float):
        for i, j in out:
            u = a[i, j] * x[i, j] + y[i, j]
            out[i, j] = ti.tanh(u) * ti.exp(-0.5 * x[i, j] * x[i, j]) + ti.sqrt(ti.abs(y[i, j]) + 1e-3)
            out2[i, j] = (u + bias[j]) * gain

    chain(1.5)
    assert chain.last_plan.startswith("map_tape") and "outputs=2" in chain.last_plan
    got, got2 = out.to_numpy(), out2.to_numpy()
    want = oracle.fused_map(av.ravel(), xv.ravel(), yv.ravel()).reshape(R, Cc)
    bound = oracle.fused_map_bound(av.ravel(), xv.ravel(), yv.ravel(), 2.0).reshape(R, Cc) + np.spacing(np.abs(want))
    assert (np.abs(got.astype(np.float64) - want) <= bound).all()
    want2 = ((av.astype(np.float64) * xv + yv) + bv[None, :]) * 1.5
    assert np.allclose(got2, want2, rtol=1e-6, atol=1e-6)


def test_unsupported_bodies_are_refused_not_interpreted():
    ti.init()
    f = ti.field(float, (8, 8))

    @ti.kernel
    def neighbour():
        for i, j in f:
            f[i, j] = f[j, i]          # a transposed read is not an elementwise map

    with pytest.raises(ti.LangError):
        neighbour()

    @ti.kernel
    def cubic():
        for i, j in f:
            z = ti.Vector([i * 0.1, j * 0.1])
            c = ti.Vector([0.1, 0.2])
            n = 0
            while z.norm() < 2 and n < 10:
                z = ti.Vector([z[0] * z[0] * z[0], z[1]]) + c   # not the quadratic map
                n += 1
            f[i, j] = 1 - n * 0.1

    with pytest.raises(ti.LangError):
        cubic()
    with pytest.raises(ti.LangError):
        ti.init(arch=ti.cpu)
