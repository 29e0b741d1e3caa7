"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header
declares, and rejects bad descriptors before touching a GPU."""
import ctypes as C
import os
import re

import pytest

from cssm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _built():
    if not os.path.exists(_lib.LIB_PATH):
        from cssm_b200 import build
        build.build()
    return _lib.lib()


def _header_symbols():
    txt = open(os.path.join(ROOT, "include", "cssm_b200.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(cssm_[a-z0-9_]+)\s*\(", txt)))


def test_library_exports_every_header_symbol():
    L = _built()
    syms = _header_symbols()
    assert len(syms) >= 15
    for s in syms:
        assert hasattr(L, s), f"{s} declared in the header but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == syms


def test_version_and_strerror():
    L = _built()
    assert b"sm_100a" in L.cssm_version()
    assert L.cssm_strerror(0) == b"ok"
    assert L.cssm_strerror(3) == b"unsupported field combination"


def _desc(**kw):
    d = dict(B=2, T=2, H=8, W=8, C=8, kernel_size=3, rope_mode=0, rope_base=10000.0,
             spectral_rho=0.999, gate_activation=0, short_conv_size=4, short_conv_spatial_size=3,
             gate_type=1)
    d.update(kw)
    return _lib.GatedDesc(**d)


def test_descriptor_validation_without_gpu():
    L = _built()
    assert L.cssm_gated_plan_bytes(C.byref(_desc())) > 0
    assert L.cssm_gated_workspace_bytes(C.byref(_desc())) > 0
    for bad in (dict(B=0), dict(C=6), dict(rope_mode=9), dict(gate_type=5),
                dict(short_conv_spatial_size=4), dict(H=4, W=64, kernel_size=11),
                dict(H=256, W=256)):
        d = _desc(**bad)
        assert L.cssm_gated_plan_bytes(C.byref(d)) == 0, bad
        assert L.cssm_gated_workspace_bytes(C.byref(d)) == 0, bad
    lay = _lib.GatedWsLayout()
    assert L.cssm_gated_workspace_layout(C.byref(_desc(B=0)), C.byref(lay)) == 2
    assert L.cssm_gated_workspace_layout(C.byref(_desc()), None) == 1
    assert L.cssm_gated_workspace_layout(C.byref(_desc()), C.byref(lay)) == 0
    assert lay.total == L.cssm_gated_workspace_bytes(C.byref(_desc()))
    # NULL pointers are rejected before any CUDA call
    w = _lib.GatedWeights()
    assert L.cssm_gated_forward(C.byref(_desc()), C.byref(w), None, None, None, None, 0, None) == 1


def test_workspace_layout_matches_formula():
    L = _built()
    d = _desc(B=3, T=5, H=64, W=64, C=16)
    lay = _lib.GatedWsLayout()
    assert L.cssm_gated_workspace_layout(C.byref(d), C.byref(lay)) == 0
    assert lay.xz_planar == 0
    assert lay.ctx_sum >= 3 * 5 * 32 * 64 * 64 * 4
    assert lay.gate_maps % 256 == 0 and lay.total % 256 == 0


def test_module_rejects_unsupported_fields():
    from cssm_b200 import GatedCSSM
    with pytest.raises(NotImplementedError):
        GatedCSSM(channels=8, dense_mixing=True).bind({"params": {}}, "cpu")
    with pytest.raises(NotImplementedError):
        GatedCSSM(channels=8, gate_type="channel").bind({"params": {}}, "cpu")


def test_module_param_tree_names_match_flax():
    from cssm_b200 import GatedCSSM
    m = GatedCSSM(channels=8, kernel_size=5, gate_type="factored")
    names = set(m.param_shapes(16, 16))
    assert names == {"in_proj", "kernel", "out_proj", "short_conv_spatial", "short_conv_temporal",
                     "delta_proj_h", "delta_proj_w", "B_proj_h", "B_proj_w", "C_proj_h", "C_proj_w"}
    m = GatedCSSM(channels=8, kernel_size=5, short_conv_size=0, short_conv_spatial_size=0)
    assert set(m.param_shapes(16, 16)) == {"in_proj", "kernel", "out_proj", "delta_proj", "B_proj",
                                           "C_proj"}
    assert m.param_shapes(16, 16)["delta_proj"]["kernel"] == (8, 16 * 9)
