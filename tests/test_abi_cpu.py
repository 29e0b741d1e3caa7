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


def _gdn_desc(**kw):
    d = dict(B=2, T=3, H=8, W=8, C=8, delta_key_dim=4, kernel_size=3, rope_mode=0, rope_base=10000.0,
             spectral_rho=0.999, gate_type=1, short_conv_size=0, output_norm=1, use_input_gates=0,
             output_gate_act=0, use_spectral_l2_norm=1, qkv_conv_size=1, no_spectral_clamp=0)
    d.update(kw)
    return _lib.GdnDesc(**d)


def test_last_frame_and_static_entry_points_validate_without_gpu():
    L = _built()
    w = _lib.GatedWeights()
    # NULL pointers: rejected before any CUDA call
    assert L.cssm_gated_forward_last(C.byref(_desc()), C.byref(w), None, None, None, None, 0, None) == 1
    gw = _lib.GdnWeights()
    assert L.cssm_gdn_forward_last(C.byref(_gdn_desc()), C.byref(gw), None, None, None, None, 0, None) == 1
    # the static-image path refuses descriptors the reference would assert on
    for bad in (dict(short_conv_size=4), dict(use_input_gates=1), dict(rope_mode=1)):
        assert L.cssm_gdn_forward_static_image(C.byref(_gdn_desc(**bad)), C.byref(gw), None, None, None,
                                               None, 0, None) == 3, bad
    assert L.cssm_gdn_forward_static_image(C.byref(_gdn_desc()), C.byref(gw), None, None, None,
                                           None, 0, None) == 1


def test_nogate_descriptor_validation_without_gpu():
    L = _built()
    d = _lib.NoGateDesc(2, 3, 8, 8, 8, 3, 0.999)
    assert L.cssm_nogate_plan_bytes(C.byref(d)) >= 8 * 8 * 5 * 8
    assert L.cssm_nogate_workspace_bytes(C.byref(d)) == 2 * 3 * 2 * 8 * 8 * 8 * 4
    assert L.cssm_nogate_plan_bytes(C.byref(_lib.NoGateDesc(2, 3, 8, 8, 6, 3, 0.999))) == 0     # C % 4
    assert L.cssm_nogate_plan_bytes(C.byref(_lib.NoGateDesc(0, 3, 8, 8, 8, 3, 0.999))) == 0
    w = _lib.NoGateWeights()
    assert L.cssm_nogate_forward(C.byref(d), C.byref(w), None, None, None, None, 0, None) == 1


def test_additive_descriptor_validation_without_gpu():
    L = _built()

    def desc(**kw):
        f = dict(B=2, T=3, H=8, W=8, C=8, kernel_size=3, rope_mode=0, rope_base=10000.0,
                 spectral_rho=0.999, gate_type=0, single_state=1, goom_floor=1)
        f.update(kw)
        return _lib.AdditiveDesc(**f)
    d = desc()
    assert L.cssm_additive_plan_bytes(C.byref(d)) >= 8 * 8 * 5 * 8
    assert L.cssm_additive_workspace_bytes(C.byref(d)) >= 2 * 3 * 2 * 8 * 8 * 8 * 4
    assert L.cssm_additive_plan_bytes(C.byref(desc(gate_type=2))) > L.cssm_additive_plan_bytes(C.byref(d))
    for bad in (desc(single_state=0), desc(gate_type=3), desc(C=6), desc(B=0), desc(goom_floor=2),
                desc(rope_mode=9)):
        assert L.cssm_additive_plan_bytes(C.byref(bad)) == 0
        assert L.cssm_additive_workspace_bytes(C.byref(bad)) == 0
    w = _lib.AdditiveWeights()
    assert L.cssm_additive_forward(C.byref(d), C.byref(w), None, None, None, None, 0, None) == 1
    assert L.cssm_additive_forward(C.byref(desc(single_state=0)), C.byref(w), None, None, None, None,
                                   0, None) == 3


def test_additive_module_rejects_unbuilt_variants():
    from cssm_b200 import AdditiveCSSM
    with pytest.raises(NotImplementedError):
        AdditiveCSSM(channels=8).init(0, (1, 2, 8, 8, 8))                      # 3-state default
    with pytest.raises(NotImplementedError):
        AdditiveCSSM(channels=8, single_state=True, gate_type="low_rank").init(0, (1, 2, 8, 8, 8))
    pc = AdditiveCSSM(channels=8, single_state=True, gate_type="channel").init(0, (1, 2, 8, 8, 8))["params"]
    assert pc["d_X"]["kernel"].shape == (8, 8) and pc["B_X"]["kernel"].shape == (1, 1, 8, 8)
    with pytest.raises(NotImplementedError):
        AdditiveCSSM(channels=8, single_state=True, learned_init=True).init(0, (1, 2, 8, 8, 8))
    m = AdditiveCSSM(channels=8, single_state=True, gate_type="factored", kernel_size=5)
    p = m.init(0, (1, 2, 8, 6, 8))["params"]
    assert p["d_X_h"]["kernel"].shape == (8, 8) and p["C_gate_w"]["kernel"].shape == (8, 4)
    assert m._floor() == 1 and AdditiveCSSM(channels=8, single_state=True, scan_mode="pallas")._floor() == 0


def test_deltanet_descriptor_validation_without_gpu():
    L = _built()

    def desc(**kw):
        f = dict(B=2, T=3, H=8, W=8, C=8, kernel_size=3, rope_mode=0, rope_base=10000.0,
                 spectral_rho=0.999, gate_type=1, goom_floor=1)
        f.update(kw)
        return _lib.DeltaNetDesc(**f)
    d = desc()
    assert L.cssm_deltanet_plan_bytes(C.byref(d)) >= 8 * 8 * 5 * 8
    assert L.cssm_deltanet_workspace_bytes(C.byref(d)) >= 2 * 3 * 3 * 8 * 8 * 8 * 4
    for bad in (desc(gate_type=3), desc(C=6), desc(T=0), desc(goom_floor=-1), desc(rope_mode=9),
                desc(H=128, W=128)):                     # plane too large for one CTA's shared memory
        assert L.cssm_deltanet_plan_bytes(C.byref(bad)) == 0
    w = _lib.DeltaNetWeights()
    assert L.cssm_deltanet_forward(C.byref(d), C.byref(w), None, None, None, None, 0, None) == 1
    assert L.cssm_deltanet_workspace_bytes(C.byref(desc(gate_type=2))) > L.cssm_deltanet_workspace_bytes(C.byref(d))
    assert L.cssm_deltanet_plan_bytes(C.byref(desc(gate_type=2, H=7, W=7, kernel_size=3))) > 0
    from cssm_b200 import DeltaNetCSSM
    with pytest.raises(NotImplementedError):
        DeltaNetCSSM(channels=8, gate_type="scalar").init(0, (1, 2, 8, 8, 8))
    pc = DeltaNetCSSM(channels=8).init(0, (1, 2, 8, 8, 8))["params"]      # default gate_type 'channel'
    assert pc["alpha"]["kernel"].shape == (8, 8) and pc["C_gate"]["kernel"].shape == (1, 1, 8, 8)
    p = DeltaNetCSSM(channels=8, gate_type="factored").init(0, (1, 2, 8, 6, 8))["params"]
    assert p["qkv_proj"]["kernel"].shape == (8, 24) and p["B_v_w"]["kernel"].shape == (8, 4)


def _simple_desc(**kw):
    d = dict(B=2, T=3, Hin=16, Win=16, Cin=1, image_input=1, stem_mode=0, stem_layers=1, embed_dim=8,
             block=0, pool_type=1, readout_norm=0, num_classes=2)
    d.update(kw)
    return _lib.SimpleDesc(**d)


def test_simple_model_descriptor_validation_without_gpu():
    L = _built()
    bd = _desc(B=2, T=3, H=8, W=8, C=8)
    n = L.cssm_simple_workspace_bytes(C.byref(_simple_desc()), C.byref(bd))
    assert n > L.cssm_gated_workspace_bytes(C.byref(bd))
    assert L.cssm_simple_host_workspace_bytes(C.byref(_simple_desc()), C.byref(bd)) > n
    # the block descriptor must describe the stem's output
    assert L.cssm_simple_workspace_bytes(C.byref(_simple_desc()), C.byref(_desc(B=2, T=3, H=16, W=16, C=8))) == 0
    assert L.cssm_simple_workspace_bytes(C.byref(_simple_desc(stem_layers=2)), C.byref(bd)) == 0
    assert L.cssm_simple_workspace_bytes(C.byref(_simple_desc(Hin=15, Win=15)), C.byref(bd)) == n      # ceil(15/2) = 8
    for bad in (dict(embed_dim=128), dict(embed_dim=6), dict(stem_mode=2), dict(stem_layers=0),
                dict(pool_type=2), dict(num_classes=0), dict(block=3)):
        assert L.cssm_simple_workspace_bytes(C.byref(_simple_desc(**bad)), C.byref(bd)) == 0, bad
    # a block descriptor the block entry points reject (unknown gate type) is rejected here too
    assert L.cssm_simple_workspace_bytes(C.byref(_simple_desc()), C.byref(_desc(B=2, T=3, H=8, W=8, C=8, gate_type=5))) == 0
    w = _lib.SimpleWeights()
    assert L.cssm_simple_forward(C.byref(_simple_desc()), C.byref(w), C.byref(bd), None, None, None,
                                 None, None, 0, 0, None) == 1
    assert L.cssm_simple_stem(C.byref(_simple_desc(embed_dim=128)), C.byref(w), None, None, None, 0, None) == 3
