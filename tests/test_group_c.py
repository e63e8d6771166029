"""The multi-GPU step driven from plain C through include/vrhi.h only (tests/c/group_gather_test.c):
one process per GPU, three back-to-back steps of the image gather with changing data and no barrier
between them, each compared bit for bit with the image one rank computes alone, plus the library's
all-reduce.  Without a GPU the program is only compiled and linked (the header is valid C and every
entry point it uses is exported)."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIBDIR = os.path.join(ROOT, "vernondsl_b200")


def build(tmp_path) -> str:
    from vernondsl_b200 import _lib

    _lib.lib()  # raises if libvrhi.so has not been built
    exe = str(tmp_path / "group_gather_test")
    cmd = ["gcc", "-O2", "-Wall", "-Werror", "-std=gnu11", "-I", os.path.join(ROOT, "include"),
           os.path.join(HERE, "c", "group_gather_test.c"), "-o", exe, "-L", LIBDIR, "-lvrhi", f"-Wl,-rpath,{LIBDIR}"]
    out = subprocess.run(cmd, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    return exe


def test_c_program_compiles_and_links(tmp_path):
    assert os.path.exists(build(tmp_path))


@pytest.mark.gpu
@pytest.mark.parametrize("ranks,squeeze", [(1, "0"), (2, "0"), (2, "1"), (4, "0"), (4, "1")])
def test_c_program_gathers_bit_exact(tmp_path, ranks, squeeze):
    """squeeze = "1": the counts cross NVLink as bytes, granules with counts of 255 and more in full (the
    default from five ranks on); "0": as uint16 by the copy engines."""
    exe = build(tmp_path)
    out = subprocess.run([exe, str(ranks)], capture_output=True, text=True, timeout=180, env=dict(os.environ, VRHI_EXCHANGE_SQUEEZE=squeeze))
    if out.returncode == 77:
        pytest.skip(f"needs {ranks} GPUs")
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    assert out.stdout.count("gathered bit-exact") == ranks
