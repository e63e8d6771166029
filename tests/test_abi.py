"""CPU: the C-ABI library loads, exports every symbol include/vrhi.h declares, and its host-only
entry points (vocabulary, registry, partition planner, error reporting) behave.  No kernel is
launched here."""
import ctypes as C
import os
import re

import pytest

from vernondsl_b200 import _lib as L
from vernondsl_b200 import ops

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vrhi.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"VRHI_API\s+[\w\s\*]+?\b(vrhi_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 50
    raw = C.CDLL(L.LIB_PATH)
    missing = [n for n in names if not hasattr(raw, n)]
    assert not missing, missing
    # and the Python binding declares a prototype for each of them
    assert sorted(L.PROTOTYPES) == names


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", os.path.join(ROOT, "vernondsl_b200", "no_such_lib.so"))
    with pytest.raises(ImportError, match="no fallback"):
        L.lib()


def test_semantic_vocabulary_matches_reference_strings():
    # VernonToSpirv.cpp:44-55 and color.mlir:9
    for k, s in enumerate(["input", "output", "uniform", "uniform_constant", "storage_buffer", "image", "varying"]):
        v = C.c_int(-1)
        assert L.lib().vrhi_arg_class_from_semantic(s.encode(), C.byref(v)) == L.OK
        assert v.value == k
        assert L.lib().vrhi_arg_class_name(k).decode() == s
    v = C.c_int()
    assert L.lib().vrhi_arg_class_from_semantic(b"push_constant", C.byref(v)) == L.ERR_NOT_FOUND
    assert b"push_constant" in L.lib().vrhi_last_error()
    assert L.lib().vrhi_arg_class_name(99) is None


def test_operator_registry():
    names = ops.op_names()
    for want in ["escape_time", "fused_map", "map_tape", "row_sum", "row_max", "row_softmax", "row_stats_softmax",
                 "col_sum", "mse_tanh_fwd", "mse_tanh_bwd", "fp32_probe", "vertex_transform", "flat_color"]:
        assert want in names
        assert names[ops.op_id(want)] == want
    with pytest.raises(L.VrhiError) as e:
        ops.op_id("no_such_kernel")
    assert e.value.status == L.ERR_NOT_FOUND
    sig = C.c_char_p()
    assert L.lib().vrhi_op_signature(ops.op_id("escape_time"), C.byref(sig)) == L.OK
    assert b"vrhi_escape_params" in sig.value
    # launching on a NULL stream is refused before any CUDA call
    assert L.lib().vrhi_op_launch(None, 0, None, 0, None, 0) == L.ERR_INVALID


def test_null_handles_are_rejected_or_ignored():
    lib = L.lib()
    for fn in ("vrhi_device_destroy", "vrhi_buffer_destroy", "vrhi_stream_destroy", "vrhi_event_destroy", "vrhi_graph_destroy"):
        assert getattr(lib, fn)(None) == L.OK
    assert lib.vrhi_device_synchronize(None) == L.ERR_INVALID
    assert lib.vrhi_stream_synchronize(None) == L.ERR_INVALID
    assert lib.vrhi_buffer_size(None, None) == L.ERR_INVALID
    assert lib.vrhi_version() == 100


@pytest.mark.parametrize("total,chunk,world", [(16384, 128, 8), (16384, 128, 1), (1080, 128, 4), (1080, 7, 3), (5, 128, 8), (1, 1, 2)])
def test_cyclic_row_partition_covers_every_row_once(total, chunk, world):
    seen = [0] * total
    owned = 0
    for rank in range(world):
        p = ops.partition_rows(total, world, rank, L.PART_CYCLIC, chunk)
        assert (p.chunk_rows, p.chunk_first, p.chunk_step) == (chunk, rank, world)
        rows = 0
        for k in range(p.chunk_count):
            c = p.chunk_first + k * p.chunk_step
            for r in range(c * chunk, min(total, (c + 1) * chunk)):
                seen[r] += 1
                rows += 1
        assert rows == p.rows_owned
        owned += rows
    assert owned == total and set(seen) == {1}


@pytest.mark.parametrize("total,chunk,world", [(16384, 0, 8), (1080, 0, 4), (1080, 128, 4), (5, 0, 8), (7, 2, 3)])
def test_contiguous_row_partition_covers_every_row_once(total, chunk, world):
    seen = [0] * total
    for rank in range(world):
        p = ops.partition_rows(total, world, rank, L.PART_CONTIGUOUS, chunk)
        assert p.chunk_count in (0, 1)
        if p.chunk_count:
            r0 = p.chunk_first * p.chunk_rows
            for r in range(r0, min(total, r0 + p.chunk_rows)):
                seen[r] += 1
            assert p.rows_owned == min(total, r0 + p.chunk_rows) - r0
        else:
            assert p.rows_owned == 0
    assert set(seen) == {1}


def test_leading_axis_partition():
    for n, world in [(2 ** 28, 8), (10, 3), (2, 4), (0, 2)]:
        spans = [ops.partition_leading(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == n
        for (b0, c0), (b1, _) in zip(spans, spans[1:]):
            assert b0 + c0 == b1
        assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(L.VrhiError):
        ops.partition_leading(10, 2, 2)
    with pytest.raises(L.VrhiError):
        ops.partition_rows(10, 0, 0)


def test_struct_layouts_match_the_header():
    # sizes a C compiler gives the structs of include/vrhi.h (checked against a compiled probe in CI is
    # not possible without a host compiler run; these are the natural-alignment sizes)
    assert C.sizeof(L.Arg) == 32
    assert C.sizeof(L.EscapeParams) == 84
    assert C.sizeof(L.MapParams) == 16
    assert C.sizeof(L.RowsParams) == 24
    assert C.sizeof(L.MseParams) == 32
    assert C.sizeof(L.TapeInstr) == 12
    assert C.sizeof(L.TapeParams) == 4 * 4 + 16 + 12 + 16 + 12 * 64 + 4 + 4 + 4  # flags, colsum_mask, trailing pad to 8
    assert C.sizeof(L.RowPartition) == 24



def test_group_and_exchange_entry_points_reject_null_handles_without_a_device():
    """The multi-GPU entry points validate their handles before they touch CUDA: NULL is an error for
    everything that uses a group or an exchange, and accepted (ignored) by the destroying functions."""
    lib = L.lib()
    out = C.c_void_p()
    null_cb = C.cast(None, L.ALLGATHER_FN)
    assert lib.vrhi_group_create(None, 2, 0, null_cb, None, C.byref(out)) == L.ERR_INVALID
    assert lib.vrhi_group_destroy(None) == L.OK
    assert lib.vrhi_exchange_destroy(None) == L.OK
    assert lib.vrhi_group_info(None, None, None) == L.ERR_INVALID
    assert lib.vrhi_group_set_wait_ms(None, 10) == L.ERR_INVALID
    assert lib.vrhi_group_all_reduce_sum_f32(None, None, 0, 1, None) == L.ERR_INVALID
    assert lib.vrhi_exchange_create(None, None, 16, 16, 1, C.byref(out)) == L.ERR_INVALID
    assert lib.vrhi_exchange_planes(None, None, None) == L.ERR_INVALID
    assert lib.vrhi_exchange_publish(None, None, 0, 1, 1) == L.ERR_INVALID
    assert lib.vrhi_exchange_complete(None, None) == L.ERR_INVALID
    assert lib.vrhi_exchange_check(None) == L.ERR_INVALID
    assert lib.vrhi_exchange_launch_count(None, None) == L.ERR_INVALID
    assert b"NULL" in lib.vrhi_last_error()


def test_the_header_is_valid_c_and_declares_what_the_library_exports(tmp_path):
    """include/vrhi.h compiles as C11 with warnings as errors, and every VRHI_API function it declares is a
    symbol of libvrhi.so (the binding table of the Python package is checked against the library elsewhere;
    this checks the header against the binding table)."""
    import re
    import subprocess

    header = os.path.join(ROOT, "include", "vrhi.h")
    src = tmp_path / "probe.c"
    src.write_text('#include "vrhi.h"\nint main(void) { return (int)sizeof(vrhi_escape_params) == 0; }\n')
    out = subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.dirname(header), "-c", str(src), "-o",
                          str(tmp_path / "probe.o")], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    declared = set(re.findall(r"VRHI_API\s+[^;(]*?\b(vrhi_\w+)\s*\(", open(header).read()))
    assert declared and declared == set(L.PROTOTYPES), (declared ^ set(L.PROTOTYPES))
