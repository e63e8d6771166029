"""GPU: device, buffer, stream and event handles of the C ABI."""
import numpy as np
import pytest

import vernondsl_b200 as vd
from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

pytestmark = pytest.mark.gpu


def test_device_properties(dev):
    assert vd.Device.count() >= 1
    assert dev.props.cc_major >= 10 and dev.sm_count > 0 and dev.sm_clock_khz > 0
    assert dev.props.total_mem_bytes > (1 << 30)


def test_upload_download_fill_roundtrip(dev, stream):
    a = np.arange(1000, dtype=np.uint32)
    b = dev.from_numpy(a, L.STORAGE_BUFFER, stream=stream)
    stream.synchronize()
    assert np.array_equal(b.download(), a)
    b.fill(0, offset=16, nbytes=32)
    got = b.download()
    assert (got[4:12] == 0).all() and got[3] == 3 and got[12] == 12
    with pytest.raises(L.VrhiError) as e:
        b.download(np.empty(2000, np.uint32))
    assert e.value.status == L.ERR_SIZE
    b.close()


def test_allocation_limit_reports_oom(dev):
    base = dev.allocated()
    dev.set_alloc_limit(base + (1 << 20))
    try:
        ok = dev.buffer(1 << 19)
        with pytest.raises(L.VrhiError) as e:
            dev.buffer(1 << 20)
        assert e.value.status == L.ERR_OOM
        ok.close()
        assert dev.allocated() == base
    finally:
        dev.set_alloc_limit(0)


def test_events_time_a_kernel_and_count_launches(dev, stream):
    out = dev.empty(4, np.float32)
    e0, e1 = dev.event(), dev.event()
    n0 = stream.launch_count()
    e0.record(stream)
    ops.fp32_probe(stream, out, ffma_per_thread=64 * 1000)
    e1.record(stream)
    e1.synchronize()
    assert e0.elapsed_ms(e1) > 0
    assert stream.launch_count() == n0 + 1
    e0.close()
    e1.close()
    out.close()


def test_wrapped_torch_tensor_and_stream(dev):
    import torch

    t = torch.zeros(64, 64, dtype=torch.int32, device="cuda:0")
    img = dev.wrap_tensor(t, L.IMAGE)
    s = dev.wrap_stream(torch.cuda.current_stream().cuda_stream)
    ops.escape_time(s, img, ops.escape_params(L.MANDELBROT, 64, 64, -2.0, -1.5, 3 / 64, 3 / 64, max_iter=40))
    s.check()
    host = t.cpu().numpy().astype(np.uint32)
    assert host.max() == 40 and host.min() <= 1
    view = img.as_tensor(np.uint32, (64, 64))
    assert view.data_ptr() == t.data_ptr() and torch.equal(view, t)
    s.close()
    img.close()


def test_shapes_whose_byte_count_wraps_are_refused_before_any_launch(dev, stream):
    """rows * cols * 4 wraps in 64 bits for shapes like 2^40 x 2^24 (2^66 bytes -> 0) and would then pass a
    size check against a tiny buffer.  Every operator that takes a [rows][cols] shape must refuse such
    a shape (VRHI_ERR_SIZE) before it launches anything."""
    import vernondsl_b200 as vd
    from vernondsl_b200 import ops

    small = dev.empty(1024, np.float32)
    vec = dev.empty(1024, np.float32)
    before = stream.launch_count()
    for rows, cols in ((1 << 40, 1 << 24), (1 << 39, 1 << 26)):
        for call in (lambda: ops.row_sum(stream, small, vec, rows, cols),
                     lambda: ops.row_softmax(stream, small, small, rows, cols),
                     lambda: ops.col_sum(stream, small, vec, rows, cols),
                     lambda: ops.mse_tanh_fwd(stream, small, small, vec, small, vec, rows, min(cols, 1 << 30)),
                     lambda: ops.mse_tanh_bwd(stream, small, small, vec, small, small, small, vec, rows, min(cols, 1 << 30))):
            with pytest.raises(vd.VrhiError) as err:
                call()
            assert err.value.status == L.ERR_SIZE
        t = ops.Tape(1)
        t.output(t.op("neg", t.input(0)))
        with pytest.raises(vd.VrhiError) as err:
            ops.map_tape(stream, t, [small], [small], rows, cols)
        assert err.value.status == L.ERR_SIZE
    assert stream.launch_count() == before
    small.close()
    vec.close()
