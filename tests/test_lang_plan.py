"""CPU: what the front end lowers a kernel to, inspected without a device (``ti.plan_only()``).

The reference's program (fractal.py:5-33) must become ONE escape_time launch whose parameter block
says exactly what the program says: which index feeds the real axis, the view window, c, the
escape test with its literal bound, the step limit and the colour map.  An elementwise body must
become one tape whose operations, evaluated in numpy here, give the body's own expression."""
import numpy as np
import pytest

import vernondsl_b200.lang as ti
from vernondsl_b200 import _lib as L

f32 = np.float32


def test_the_reference_program_lowers_to_one_escape_time_launch():
    n = 320                                              # fractal.py:7
    with ti.plan_only():
        pixels = ti.field(dtype=float, shape=(n * 2, n))     # fractal.py:8

        @ti.func
        def complex_sqr(z):                              # fractal.py:11-13
            return ti.Vector([z[0] ** 2 - z[1] ** 2, z[1] * z[0] * 2])

        @ti.kernel
        def paint(t: float):                             # fractal.py:16-25
            for i, j in pixels:
                c = ti.Vector([-0.8, ti.cos(t) * 0.2])
                z = ti.Vector([i / n - 1, j / n - 0.5]) * 2
                iterations = 0
                while z.norm() < 20 and iterations < 50:
                    z = complex_sqr(z) + c
                    iterations += 1
                pixels[i, j] = 1 - iterations * 0.02

        for frame in (0, 7, 1000):                       # fractal.py:30-31: a new uniform, nothing else changes
            t = frame * 0.03
            paint(t)
            p = paint.last_params
            assert pixels.buffer is None
            assert paint.last_plan == "escape_time kind=julia 320x640 transposed=True"
            assert (p.kind, p.mode, p.test, p.output) == (L.JULIA, L.EXACT, L.TEST_NORM_GE, L.OUT_COLOR_F32)
            assert (p.width, p.height, p.max_iter) == (n, 2 * n, 50)      # rows follow the first index i
            assert p.flags == 2                                           # transposed: the real part follows the row
            assert (p.chunk_rows, p.chunk_count) == (0, 0)                # the whole image
            # real = (i/n - 1)*2 = -2 + i*(2/n) along the rows (y0, dy); imaginary = -1 + j*(2/n) along the columns
            assert (f32(p.y0), f32(p.dy), f32(p.x0), f32(p.dx)) == (f32(-2.0), f32(2.0 / n), f32(-1.0), f32(2.0 / n))
            assert f32(p.cr) == f32(-0.8)
            assert f32(p.ci) == f32(np.cos(f32(t))) * f32(0.2)            # evaluated on the host in binary32
            assert f32(p.bound) == f32(20.0) and f32(p.color_scale) == f32(0.02)
    with pytest.raises(ti.LangError):
        pixels.to_numpy()                                # a planned field holds nothing


def test_mandelbrot_into_an_integer_field_lowers_untransposed():
    W, H, N = 200, 120, 300
    with ti.plan_only():
        img = ti.field(dtype=int, shape=(H, W))

        @ti.kernel
        def mandel():
            for r, c in img:
                k = ti.Vector([c * (3.5 / W) - 2.5, r * (2.0 / H) - 1.0])
                z = ti.Vector([0.0, 0.0])
                m = 0
                while z.norm_sqr() <= 4 and m < N:
                    z = ti.Vector([z[0] * z[0] - z[1] * z[1], 2 * z[0] * z[1]]) + k
                    m += 1
                img[r, c] = m

        mandel()
    p = mandel.last_params
    assert (p.kind, p.test, p.output, p.flags) == (L.MANDELBROT, L.TEST_NORM2_GT, L.OUT_COUNT_U32, 0)
    assert (p.width, p.height, p.max_iter) == (W, H, N)
    assert (f32(p.x0), f32(p.dx), f32(p.y0), f32(p.dy)) == (f32(-2.5), f32(3.5 / W), f32(-1.0), f32(2.0 / H))
    assert f32(p.bound) == f32(4.0)


def evaluate(tape, inputs):
    """The tape's operations in numpy binary64 (only the operations these tests use)."""
    names = {v: k for k, v in L.T.items()}
    fn = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide, "neg": np.negative, "abs": np.abs,
          "square": np.square, "sqrt": np.sqrt, "exp": np.exp, "tanh": np.tanh, "max": np.maximum, "min": np.minimum,
          "cos": np.cos, "sin": np.sin}
    vals = list(inputs)
    for op, a, b, c, imm in tape.instr:
        name = names[op]
        if name == "const":
            vals.append(np.float64(imm))
        elif name == "fma":
            vals.append(vals[a] * vals[b] + vals[c])
        elif name in ("add", "sub", "mul", "div", "max", "min"):
            vals.append(fn[name](vals[a], vals[b]))
        else:
            vals.append(fn[name](vals[a]))
    return [vals[k] for k in tape.outputs]


def test_an_elementwise_body_lowers_to_one_tape_that_computes_the_body():
    R, Cc = 6, 8
    rng = np.random.default_rng(3)
    av, xv, yv = rng.uniform(-1, 1, (R, Cc)), rng.standard_normal((R, Cc)), rng.standard_normal((R, Cc))
    bv = rng.standard_normal(Cc)
    with ti.plan_only():
        a, x, y, out, out2 = (ti.field(float, (R, Cc)) for _ in range(5))
        bias = ti.field(float, (Cc,))

        @ti.kernel
        def chain(gain: float):
            for i, j in out:
                u = a[i, j] * x[i, j] + y[i, j]
                out[i, j] = ti.tanh(u) * ti.exp(-0.5 * x[i, j] * x[i, j]) + ti.sqrt(ti.abs(y[i, j]) + 1e-3)
                out2[i, j] = (u + bias[j]) * gain

        chain(1.5)
    tape = chain.last_tape
    assert chain.last_plan.startswith("map_tape inputs=4 outputs=2")
    assert tape.n_inputs == 4 and tape.row_mask == 0b1000 and tape.col_mask == 0 and len(tape.outputs) == 2
    assert len(tape.instr) <= L.TAPE_MAX_INSTR
    got, got2 = evaluate(tape, [av, xv, yv, bv[None, :]])
    u = av * xv + yv
    assert np.allclose(got, np.tanh(u) * np.exp(-0.5 * xv * xv) + np.sqrt(np.abs(yv) + f32(1e-3)), rtol=1e-12)
    assert np.allclose(got2, (u + bv[None, :]) * 1.5, rtol=1e-12)
    # u is computed once: the two stores share it
    names = {v: k for k, v in L.T.items()}
    assert sum(1 for op, *_ in tape.instr if names[op] == "tanh") == 1
    p = tape.params(R, Cc)
    assert (p.n_inputs, p.n_outputs, p.rows, p.cols, p.row_vector_mask) == (4, 2, R, Cc, 0b1000)


def test_bodies_outside_the_two_shapes_are_refused_while_planning_too():
    with ti.plan_only():
        f = ti.field(float, (8, 8))

        @ti.kernel
        def neighbour():
            for i, j in f:
                f[i, j] = f[j, i]

        @ti.kernel
        def cubic():
            for i, j in f:
                z = ti.Vector([i * 0.1, j * 0.1])
                c = ti.Vector([0.1, 0.2])
                m = 0
                while z.norm() < 2 and m < 10:
                    z = ti.Vector([z[0] * z[0] * z[0], z[1]]) + c
                    m += 1
                f[i, j] = 1 - m * 0.1

        @ti.kernel
        def wrong_test():
            for i, j in f:
                z = ti.Vector([i * 0.1, j * 0.1])
                c = ti.Vector([0.1, 0.2])
                m = 0
                while z.norm() <= 2 and m < 10:          # only `norm() < R` and `norm_sqr() <= R` are stated exactly
                    z = ti.Vector([z[0] ** 2 - z[1] ** 2, z[1] * z[0] * 2]) + c
                    m += 1
                f[i, j] = 1 - m * 0.1

        for k in (neighbour, cubic, wrong_test):
            with pytest.raises(ti.LangError):
                k()
