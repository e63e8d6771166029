"""GPU: the per-element maps of the reference's shader input file (color.mlir) as CUDA kernels over
arrays: vec3 -> vec4 extension, three chained 4x4 matrix-vector products per vertex, flat colour
per fragment of a headless pixel buffer.  Oracle: the same arithmetic in binary64."""
import numpy as np
import pytest

import oracle
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu


def matrices(seed):
    rng = np.random.default_rng(seed)
    model = np.eye(4, dtype=np.float32)
    model[:3, :3] = rng.standard_normal((3, 3)).astype(np.float32)
    model[:3, 3] = rng.standard_normal(3).astype(np.float32)
    view = np.eye(4, dtype=np.float32)
    view[:3, 3] = [0.0, -0.5, -4.0]
    f, near, far = 1.3, 0.1, 50.0
    proj = np.zeros((4, 4), dtype=np.float32)
    proj[0, 0] = proj[1, 1] = f
    proj[2, 2], proj[2, 3] = (far + near) / (near - far), 2 * far * near / (near - far)
    proj[3, 2] = -1.0
    return model, view, proj


@pytest.mark.parametrize("n", [1, 7, 1000, 300001])
def test_vertex_transform(dev, stream, n):
    rng = np.random.default_rng(n)
    pos = rng.standard_normal((n, 3)).astype(np.float32)
    model, view, proj = matrices(n)
    P = dev.from_numpy(pos)
    M, V, J = (dev.from_numpy(m, L.UNIFORM) for m in (model, view, proj))
    out, var = dev.empty((n, 4), np.float32), dev.empty((n, 3), np.float32, L.VARYING)
    ops.vertex_transform(stream, P, M, V, J, out, var, n)
    stream.check()
    want, want_var = oracle.vertex_transform(pos, model, view, proj)
    got = out.download()
    # three chained products of O(1..10) numbers: 1e-5 relative to the largest component of each vertex
    scale = np.abs(want).max(axis=1, keepdims=True) + 1e-30
    assert (np.abs(got - want) <= 1e-5 * scale).all()
    assert np.array_equal(var.download(), want_var)          # the varying is a pass-through
    assert np.array_equal(got[:, 3] != 0, want[:, 3] != 0)   # w = -z_view: the perspective row is applied


def test_identity_matrices_give_the_extended_position(dev, stream):
    n = 513
    pos = np.random.default_rng(1).standard_normal((n, 3)).astype(np.float32)
    eye = np.eye(4, dtype=np.float32)
    P = dev.from_numpy(pos)
    M, V, J = (dev.from_numpy(eye, L.UNIFORM) for _ in range(3))
    out, var = dev.empty((n, 4), np.float32), dev.empty((n, 3), np.float32, L.VARYING)
    ops.vertex_transform(stream, P, M, V, J, out, var, n)
    stream.check()
    got = out.download()
    assert np.array_equal(got[:, :3], pos) and (got[:, 3] == 1.0).all()   # color.mlir:20-27: vec4(pos, 1.0)


def test_flat_color(dev, stream):
    w, h = 640, 360
    color = np.array([0.25, 0.5, 0.75], dtype=np.float32)
    Cc = dev.from_numpy(color, L.UNIFORM)
    frag = dev.empty((h * w, 4), np.float32, L.IMAGE)
    frag.fill(0xFF)
    ops.flat_color(stream, Cc, frag, h * w)
    stream.check()
    got = frag.download()
    assert (got == np.array([0.25, 0.5, 0.75, 1.0], dtype=np.float32)).all()   # color.mlir:51-59: vec4(color, 1.0)


def test_errors(dev, stream):
    small = dev.from_numpy(np.zeros(4, np.float32), L.UNIFORM)
    frag = dev.empty((8, 4), np.float32, L.IMAGE)
    with pytest.raises(L.VrhiError) as e:
        ops.flat_color(stream, small, frag, 9)
    assert e.value.status == L.ERR_SIZE
    with pytest.raises(L.VrhiError) as e:
        ops.flat_color(stream, small, small, 1)   # a UNIFORM buffer cannot be written
    assert e.value.status == L.ERR_INVALID
