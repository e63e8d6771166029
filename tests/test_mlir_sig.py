"""CPU: kernel signatures with vernon.semantic attributes -> runtime argument classes."""
import os

import pytest

from vernondsl_b200 import _lib as L
from vernondsl_b200 import mlir_sig

# A module in the same textual form as the reference's shader input (func.func with per-argument
# and per-result `vernon.semantic` attributes); written for this test, not taken from it.
EXAMPLE = r"""
module {
  // a skinning-style vertex stage
  func.func @skin_main(%p: tensor<3xf32> {vernon.semantic = "input"},
                       %bones: tensor<16x4x4xf32> {vernon.semantic = "storage_buffer"},
                       %world: tensor<4x4xf32> {vernon.semantic = "uniform"},
                       %lut: tensor<256xf32> {vernon.semantic="uniform_constant"},
                       %plain: f32)
                   -> (tensor<4xf32> {vernon.semantic="output"},
                       tensor<2xf32> {vernon.semantic = "varying"}) {
    %z = arith.constant 0.0 : f32
    return
  }
  func.func @shade_main(%albedo: tensor<8x8xf32> {vernon.semantic = "image"},
                        %uv: tensor<2xf32> {vernon.semantic = "varying"}) -> tensor<4xf32> {
    return
  }
}
"""


def test_example_module():
    sigs = mlir_sig.parse_signatures(EXAMPLE)
    assert [s.name for s in sigs] == ["skin_main", "shade_main"]
    skin, shade = sigs
    assert [a.name for a in skin.args] == ["%p", "%bones", "%world", "%lut", "%plain"]
    assert [a.semantic for a in skin.args] == ["input", "storage_buffer", "uniform", "uniform_constant", None]
    assert [a.arg_class for a in skin.args] == [L.INPUT, L.STORAGE_BUFFER, L.UNIFORM, L.UNIFORM_CONSTANT, None]
    assert skin.args[1].type == "tensor<16x4x4xf32>" and skin.args[1].shape == (16, 4, 4) and skin.args[1].n_elements == 256
    assert [r.arg_class for r in skin.results] == [L.OUTPUT, L.VARYING]
    assert skin.results[1].shape == (2,)
    assert [a.arg_class for a in shade.args] == [L.IMAGE, L.VARYING]
    assert len(shade.results) == 1 and shade.results[0].type == "tensor<4xf32>" and shade.results[0].semantic is None


def test_unknown_semantic_is_an_error():
    bad = 'func.func @f(%a: tensor<4xf32> {vernon.semantic = "push_constant"}) { return }'
    with pytest.raises(L.VrhiError) as e:
        mlir_sig.parse_signatures(bad)
    assert e.value.status == L.ERR_NOT_FOUND


# where a checkout of the reference project lies, if anywhere: VERNON_REFERENCE_ROOT, else a `reference`
# directory beside the repository; the test is skipped where there is none (a GPU box, for instance)
_HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.environ.get("VERNON_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
REFERENCE_FILE = os.path.join(REFERENCE_ROOT, "source", "tests", "integration", "color.mlir")


@pytest.mark.skipif(not os.path.exists(REFERENCE_FILE), reason="no checkout of the reference project here")
def test_reference_shader_file():
    """The reference's own input: vertex_main (color.mlir:4-9) and frag_main (:43-45)."""
    sigs = {s.name: s for s in mlir_sig.parse_signatures(open(REFERENCE_FILE).read())}
    v, f = sigs["vertex_main"], sigs["frag_main"]
    assert [a.semantic for a in v.args] == ["input", "uniform", "uniform", "uniform"]
    assert [a.shape for a in v.args] == [(3,), (4, 4), (4, 4), (4, 4)]
    assert [r.semantic for r in v.results] == ["output", "varying"]
    assert [r.arg_class for r in v.results] == [L.OUTPUT, L.VARYING]   # `varying` is unhandled by the reference pass
    assert [a.semantic for a in f.args] == ["uniform", "varying"] and [r.semantic for r in f.results] == ["output"]
