"""GPU parity of the GDN block (through the C ABI) against the NumPy oracle (fp64 tier).
Tolerance: rel-L2 <= 1e-4 in fp32."""
import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from cssm_b200 import GatedDeltaNetCSSM

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _run(B, T, H, W, C, dk, ks, gate, rope, kt, qkvk, ig=True, norm="rms", act="silu", l2=True,
         seed=0, last=False):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_gdn_params(seed + 1, C, H, W, delta_key_dim=dk, kernel_size=ks, gate_type=gate,
                            short_conv_size=kt, qkv_conv_size=qkvk, use_input_gates=ig,
                            bias_scale=0.1, perturb_rms=True)
    ref, inter = orc.gdn_forward(p, x, delta_key_dim=dk, kernel_size=ks, rope_mode=rope,
                                 gate_type=gate, short_conv_size=kt, qkv_conv_size=qkvk,
                                 use_input_gates=ig, output_norm=norm, output_gate_act=act,
                                 use_spectral_l2_norm=l2, return_intermediates=True)
    mod = GatedDeltaNetCSSM(channels=C, delta_key_dim=dk, kernel_size=ks, rope_mode=rope,
                            gate_type=gate, short_conv_size=kt, qkv_conv_size=qkvk,
                            use_input_gates=ig, output_norm=norm, output_gate_act=act,
                            use_spectral_l2_norm=l2)
    xd = torch.from_numpy(x).cuda()
    y = mod.apply({"params": p}, xd).cpu().numpy()
    if last:
        y_last = mod.bind({"params": p})(xd, last_frame_only=True).cpu().numpy()
        return y, ref, y_last
    return y, ref


CASES = [
    # B, T, H, W, C, dk, ks, gate, rope, kt, qkv_conv
    (2, 3, 8, 8, 8, 4, 5, "factored", "mrope", 4, 5),
    (1, 4, 8, 8, 8, 2, 3, "dense", "none", 4, 1),
    (2, 2, 6, 10, 12, 3, 3, "factored", "spatiotemporal", 2, 3),
    (1, 3, 32, 32, 8, 4, 11, "factored", "mrope", 4, 1),       # 32x32 radix kernel, state on chip
    (2, 5, 32, 32, 16, 4, 11, "dense", "spatiotemporal", 4, 3),
    (2, 3, 64, 64, 8, 4, 11, "factored", "mrope", 4, 5),
    (1, 8, 64, 64, 4, 4, 11, "dense", "none", 4, 1),
    (1, 2, 64, 64, 8, 2, 11, "factored", "none", 0, 1),      # 64x64 with d_k=2: generic kernel
    (1, 2, 7, 7, 8, 4, 11, "factored", "temporal", 4, 3),    # kernel larger than the plane
    (1, 2, 64, 64, 64, 4, 11, "factored", "mrope", 4, 5),    # C = 64: tensor-core projections
    # per-head alpha/beta, 1x1-conv spatial gates ('channel', the reference default) and one
    # scalar per frame ('scalar'), on the generic, 32x32 and 64x64 recurrence kernels
    (2, 3, 8, 8, 8, 4, 5, "channel", "mrope", 4, 3),
    (1, 3, 32, 32, 16, 4, 11, "channel", "spatiotemporal", 4, 1),
    (1, 3, 64, 64, 8, 4, 11, "channel", "mrope", 4, 5),
    (1, 2, 64, 64, 64, 4, 11, "channel", "none", 0, 1),
    (2, 3, 6, 10, 12, 3, 3, "scalar", "temporal", 2, 1),
    (1, 3, 32, 32, 8, 4, 11, "scalar", "mrope", 4, 3),
    (1, 2, 64, 64, 8, 4, 11, "scalar", "none", 4, 1),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c)))
def test_block_parity(case):
    y, ref = _run(*case)
    assert np.isfinite(y).all()
    assert orc.rel_l2(y, ref) <= TOL


def test_channel_gates_without_input_gates():
    y, ref = _run(1, 3, 32, 32, 8, 4, 5, "channel", "none", 4, 1, ig=False)
    assert orc.rel_l2(y, ref) <= TOL


@pytest.mark.parametrize("kw", [dict(ig=False), dict(norm="none"), dict(act="sigmoid"),
                                dict(l2=False)], ids=str)
def test_field_variants(kw):
    y, ref = _run(1, 3, 8, 8, 8, 4, 5, "factored", "none", 4, 1, **kw)
    assert orc.rel_l2(y, ref) <= TOL
    y, ref = _run(1, 2, 64, 64, 4, 4, 5, "factored", "none", 4, 1, **kw)
    assert orc.rel_l2(y, ref) <= TOL


def test_golden_fixture():
    import os
    from tests.golden import make_golden as mg
    g = np.load(os.path.join(os.path.dirname(mg.__file__), "gdn_small.npz"))
    x, p, kw = mg.gdn_case()
    mod = GatedDeltaNetCSSM(channels=x.shape[-1], **kw)
    y = mod.apply({"params": p}, torch.from_numpy(g["x"]).cuda()).cpu().numpy()
    assert orc.rel_l2(y, g["y"]) <= TOL


def test_deterministic():
    rng = np.random.default_rng(0)
    x = torch.from_numpy(rng.standard_normal((1, 3, 64, 64, 8)).astype(np.float32)).cuda()
    mod = GatedDeltaNetCSSM(channels=8, delta_key_dim=4, gate_type="factored")
    v = mod.init(0, tuple(x.shape), bias_scale=0.1)
    y1 = mod.apply(v, x).clone()
    y2 = mod.apply(v, x).clone()
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("case", [CASES[0], CASES[1], CASES[4], CASES[5], CASES[7], CASES[9], CASES[11],
                                  CASES[12], CASES[15]],
                         ids=lambda c: "x".join(map(str, c)))
def test_last_frame_only_matches_full_forward(case):
    """cssm_gdn_forward_last equals the last frame of the full forward (generic, 32x32 and 64x64
    kernels; CUDA-core and tensor-core projections) and the oracle's last frame."""
    y, ref, y_last = _run(*case, last=True)
    assert y_last.shape == y[:, -1].shape
    assert np.isfinite(y_last).all()
    assert orc.rel_l2(y_last, y[:, -1]) <= 1e-6
    assert orc.rel_l2(y_last, ref[:, -1]) <= TOL


STATIC_CASES = [
    # B, T, H, W, C, dk, ks, gate, qkv_conv
    (2, 4, 8, 8, 8, 4, 5, "factored", 3),          # generic kernel
    (2, 6, 32, 32, 8, 4, 11, "dense", 1),          # 32x32 radix kernel
    (2, 5, 64, 64, 8, 4, 11, "factored", 5),       # 64x64 radix kernel
    (1, 3, 64, 64, 64, 4, 11, "factored", 1),      # tensor-core projections
    (1, 3, 14, 14, 8, 2, 3, "factored", 1),        # d_k = 2
]


@pytest.mark.parametrize("case", STATIC_CASES, ids=lambda c: "x".join(map(str, c)))
def test_static_image_fast_path(case):
    """4-D input through cssm_gdn_forward_static_image against the oracle of the reference's
    static-image path, which carries M_t, Delta_t and the state in bfloat16: tolerance rel-L2
    <= 2e-2 (the bf16 tolerance).  Two kernels that round at slightly different fp32 inputs may
    land on neighbouring bf16 values, so exact fp32-level agreement is not expected; the error
    against the SAME scan carried in fp64 must be of the size the oracle's own bf16 rounding
    costs."""
    B, T, H, W, C, dk, ks, gate, qkvk = case
    rng = np.random.default_rng(7)
    x = rng.standard_normal((B, H, W, C)).astype(np.float32)
    p = orc.init_gdn_params(8, C, H, W, delta_key_dim=dk, kernel_size=ks, gate_type=gate,
                            short_conv_size=0, qkv_conv_size=qkvk, use_input_gates=False,
                            bias_scale=0.1, perturb_rms=True)
    kw = dict(num_timesteps=T, delta_key_dim=dk, kernel_size=ks, gate_type=gate, qkv_conv_size=qkvk)
    ref = orc.gdn_static_forward(p, x, **kw)
    ref64 = orc.gdn_static_forward(p, x, carry="fp64", **kw)
    mod = GatedDeltaNetCSSM(channels=C, delta_key_dim=dk, kernel_size=ks, rope_mode="none",
                            gate_type=gate, short_conv_size=0, qkv_conv_size=qkvk,
                            use_input_gates=False, static_image_fast_path=True, num_timesteps=T)
    y = mod.apply({"params": p}, torch.from_numpy(x).cuda()).cpu().numpy()
    assert y.shape == x.shape and np.isfinite(y).all()
    assert orc.rel_l2(y, ref) <= 2e-2
    assert orc.rel_l2(y, ref64) <= 2.0 * orc.rel_l2(ref, ref64) + 1e-4


def test_static_image_preconditions():
    with pytest.raises(AssertionError):
        GatedDeltaNetCSSM(channels=8, delta_key_dim=4, static_image_fast_path=True, num_timesteps=4,
                          short_conv_size=4, use_input_gates=False, gate_type="factored").bind({"params": {}})
    with pytest.raises(AssertionError):
        GatedDeltaNetCSSM(channels=8, delta_key_dim=4, static_image_fast_path=True, num_timesteps=0,
                          short_conv_size=0, use_input_gates=False, gate_type="factored").bind({"params": {}})


def test_static_image_golden_fixture_on_gpu():
    """The committed fixture of the static-image path (tests/golden/gdn_static_small.npz)."""
    import os
    from tests.golden import make_golden as mg
    g = np.load(os.path.join(os.path.dirname(mg.__file__), "gdn_static_small.npz"))
    _, p, kw = mg.gdn_static_case()
    mod = GatedDeltaNetCSSM(channels=g["x"].shape[-1], delta_key_dim=4, kernel_size=kw["kernel_size"],
                            rope_mode="none", gate_type="factored", short_conv_size=0,
                            qkv_conv_size=kw["qkv_conv_size"], use_input_gates=False,
                            static_image_fast_path=True, num_timesteps=kw["num_timesteps"])
    y = mod.apply({"params": p}, torch.from_numpy(g["x"]).cuda()).cpu().numpy()
    assert orc.rel_l2(y, g["y"]) <= 2e-2
