"""Seeded random sweeps over shapes and fields of the six module mirrors on the GPU, each case
checked against the NumPy oracle (rel-L2 <= 1e-4, fp32), including the last-frame-only calls."""
import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from oracle import simple_oracle as so
from cssm_b200 import (AdditiveCSSM, DeltaNetCSSM, GatedCSSM, GatedDeltaNetCSSM, NoGateCSSM,
                       SimpleCSSM)

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _case(seed):
    rng = np.random.default_rng(seed)

    def pick(*a):
        return a[rng.integers(len(a))]

    kind = pick("gated", "gdn", "nogate", "simple", "gated", "gdn")
    size = pick("rand", "rand", "r32", "r64")
    H, W = {"r32": (32, 32), "r64": (64, 64)}.get(size, (int(rng.integers(3, 19)), int(rng.integers(3, 19))))
    B, T = int(rng.integers(1, 4)), int(rng.integers(1, 6))
    C = int(pick(4, 8, 12, 16)) if size == "rand" else int(pick(4, 8, 64))
    if C == 64:
        B, T = 1, int(rng.integers(1, 4))
    ks = int(pick(1, 3, 5, 7, 11))
    if (ks > H) != (ks > W):
        ks = 1
    rope = pick("none", "spatiotemporal", "mrope", "temporal", "spatial_only")
    gate = pick("factored", "dense")
    xd = None
    if kind == "gated":
        kt, ksp, ga = int(pick(0, 2, 4)), int(pick(0, 3, 5)), pick("softplus", "softplus", "sigmoid", "exp")
        x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
        p = orc.init_gated_params(seed, C, H, W, kernel_size=ks, gate_type=gate, short_conv_size=kt,
                                  short_conv_spatial_size=ksp, bias_scale=0.1)
        kw = dict(kernel_size=ks, rope_mode=rope, gate_type=gate, short_conv_size=kt,
                  short_conv_spatial_size=ksp)
        ref = orc.gated_forward(p, x, gate_activation_kind=ga, **kw)
        b = GatedCSSM(channels=C, gate_activation=ga, **kw).bind({"params": p})
        xd = torch.from_numpy(x).cuda()
        return [(b(xd), ref), (b(xd, last_frame_only=True), ref[:, -1])]
    if kind == "gdn":
        dk = int(pick(1, 2, 4, 4))
        if C % dk:
            dk = 4
        kt, qk, ig = int(pick(0, 2, 4)), int(pick(1, 3, 5)), bool(pick(0, 1))
        kw = dict(delta_key_dim=dk, kernel_size=ks, rope_mode=rope, gate_type=gate, short_conv_size=kt,
                  qkv_conv_size=qk, use_input_gates=ig, output_norm=pick("rms", "none"),
                  output_gate_act=pick("silu", "sigmoid"), use_spectral_l2_norm=bool(pick(1, 1, 0)))
        x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
        p = orc.init_gdn_params(seed, C, H, W, delta_key_dim=dk, kernel_size=ks, gate_type=gate,
                                short_conv_size=kt, qkv_conv_size=qk, use_input_gates=ig,
                                bias_scale=0.1, perturb_rms=True)
        ref = orc.gdn_forward(p, x, **kw)
        b = GatedDeltaNetCSSM(channels=C, **kw).bind({"params": p})
        xd = torch.from_numpy(x).cuda()
        return [(b(xd), ref), (b(xd, last_frame_only=True), ref[:, -1])]
    if kind == "nogate":
        x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
        mod = NoGateCSSM(channels=C, kernel_size=ks)
        p = mod.init(seed, x.shape, bias_scale=0.1)["params"]
        p["kernel"] = (0.3 * rng.standard_normal(p["kernel"].shape)).astype(np.float32)
        return [(mod.apply({"params": p}, torch.from_numpy(x).cuda()), orc.nogate_forward(p, x, kernel_size=ks))]
    ct, E, layers, sm = pick("gated", "gdn"), int(pick(8, 16)), int(pick(1, 2)), pick("default", "pathtracker")
    Hin, Win, Cin = int(rng.integers(6, 40)), int(rng.integers(6, 40)), int(pick(1, 3))
    img, pool, rn, seq = bool(pick(0, 1)), pick("mean", "max"), pick("pre", "post"), int(rng.integers(1, 5))
    pos = pick("none", "spatiotemporal", "mrope")
    extra = dict(delta_key_dim=4, qkv_conv_size=int(pick(1, 3))) if ct == "gdn" else {}
    m = SimpleCSSM(cssm_type=ct, embed_dim=E, kernel_size=min(ks, 7), pos_embed=pos, stem_mode=sm,
                   stem_layers=layers, pool_type=pool, readout_norm=rn, gate_type=gate, seq_len=seq,
                   num_classes=int(pick(2, 5)), **extra)
    Hf, Wf = m.feature_hw(Hin, Win)
    if (m.kernel_size > Hf) != (m.kernel_size > Wf):
        return []
    x = rng.random((B, Hin, Win, Cin) if img else (B, T, Hin, Win, Cin)).astype(np.float32)
    bkw = dict(kernel_size=m.kernel_size, rope_mode=pos, gate_type=gate, short_conv_size=4)
    if ct == "gated":
        bkw["short_conv_spatial_size"] = 3
    else:
        bkw.update(delta_key_dim=4, qkv_conv_size=extra["qkv_conv_size"])
    p = so.init_simple_params(seed, cin=Cin, embed_dim=E, H=Hf, W=Wf, num_classes=m.num_classes,
                              cssm_type=ct, stem_mode=sm, stem_layers=layers, bias_scale=0.1,
                              block_kwargs=bkw)
    ref = so.simple_forward(p, x, cssm_type=ct, seq_len=seq, stem_mode=sm, stem_layers=layers,
                            pool_type=pool, readout_norm=rn, block_kwargs=bkw)
    b = m.bind({"params": p})
    xd = torch.from_numpy(x).cuda()
    return [(b(xd), ref), (b(xd, last_frame_only=True), ref)]


@pytest.mark.parametrize("seed", range(100, 148))
def test_random_configuration(seed):
    for got, ref in _case(seed):
        got = got.cpu().numpy()
        assert np.isfinite(got).all()
        assert orc.rel_l2(got, ref) <= TOL


def _scalar_case(seed):
    """Single-state AdditiveCSSM / DeltaNetCSSM with random shape, gates, RoPE and scan mode."""
    rng = np.random.default_rng(seed)

    def pick(*a):
        return a[rng.integers(len(a))]

    kind = pick("additive", "deltanet")
    size = pick("rand", "rand", "r32", "r64")
    H, W = {"r32": (32, 32), "r64": (64, 64)}.get(size, (int(rng.integers(3, 19)), int(rng.integers(3, 19))))
    B, T = int(rng.integers(1, 4)), int(rng.integers(1, 7))
    C = int(pick(4, 8, 12, 16)) if size == "rand" else int(pick(4, 8, 64))
    if C == 64:
        B, T = 1, int(rng.integers(1, 4))
    ks = int(pick(1, 3, 5, 7, 11))
    if (ks > H) != (ks > W):
        ks = 1
    rope = pick("none", "spatiotemporal", "mrope", "temporal", "spatial_only")
    gate = pick("factored", "dense")
    mode = pick("associative", "associative", "ssd", "quadratic", "pallas")
    if pick(0, 1):
        gate = "channel"
    x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
    kw = dict(kernel_size=ks, gate_type=gate, rope_mode=rope, scan_mode=mode)
    if kind == "additive":
        p = orc.init_additive1_params(seed, C, H, W, kernel_size=ks, gate_type=gate, bias_scale=0.1)
        ref = orc.additive1_forward(p, x, **kw)
        mod = AdditiveCSSM(channels=C, single_state=True, **kw)
    else:
        p = orc.init_deltanet_params(seed, C, H, W, kernel_size=ks, gate_type=gate, bias_scale=0.1)
        p["output_proj"]["bias"][:] = 0
        ref = orc.deltanet_forward(p, x, **kw)
        mod = DeltaNetCSSM(channels=C, **kw)
    return mod.apply({"params": p}, torch.from_numpy(x).cuda()), ref


@pytest.mark.parametrize("seed", range(200, 232))
def test_random_scalar_scan_configuration(seed):
    got, ref = _scalar_case(seed)
    got = got.cpu().numpy()
    assert np.isfinite(got).all()
    assert orc.rel_l2(got, ref) <= TOL
