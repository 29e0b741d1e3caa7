"""The five blocks on input distributions that stress the arithmetic rather than the indexing:
constant planes (all spectral energy in the DC bin), zeros (the magnitude floors), an impulse, a
2 %-sparse signal, a constant plus 1e-3 noise (cancellation), values of 1e3 and of 1e-4, and a
clip whose frames after the first are zero (pure state decay).  Each against the NumPy oracle,
rel-L2 <= 1e-4 (fp32)."""
import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from cssm_b200 import AdditiveCSSM, DeltaNetCSSM, GatedCSSM, GatedDeltaNetCSSM, NoGateCSSM

pytestmark = pytest.mark.gpu
TOL = 1e-4
SHAPES = [(2, 4, 64, 64, 64), (2, 5, 32, 32, 8), (2, 3, 14, 10, 12)]
KINDS = ["const_per_channel", "zeros", "impulse", "large_1e3", "tiny_1e-4", "sparse_2pct",
         "const_plus_noise", "first_frame_only"]


def _input(kind, shape, rng):
    B, T, H, W, C = shape
    if kind == "const_per_channel":
        return np.broadcast_to(rng.standard_normal((1, 1, 1, 1, C)), shape).astype(np.float32).copy()
    if kind == "zeros":
        return np.zeros(shape, np.float32)
    if kind == "impulse":
        x = np.zeros(shape, np.float32)
        x[:, :, H // 2, W // 3, :] = 1.0
        return x
    if kind == "large_1e3":
        return (1e3 * rng.standard_normal(shape)).astype(np.float32)
    if kind == "tiny_1e-4":
        return (1e-4 * rng.standard_normal(shape)).astype(np.float32)
    if kind == "sparse_2pct":
        return (rng.standard_normal(shape) * (rng.random(shape) < 0.02)).astype(np.float32)
    if kind == "const_plus_noise":
        base = np.broadcast_to(rng.standard_normal((1, 1, 1, 1, C)), shape)
        return (base + 1e-3 * rng.standard_normal(shape)).astype(np.float32)
    x = np.zeros(shape, np.float32)
    x[:, 0] = rng.standard_normal((B, H, W, C))
    return x


def _block(name, shape, rng):
    B, T, H, W, C = shape
    ks = 5
    if name == "gated":
        kw = dict(kernel_size=ks, rope_mode="spatiotemporal", gate_type="factored", short_conv_size=4,
                  short_conv_spatial_size=3)
        p = orc.init_gated_params(1, C, H, W, kernel_size=ks, gate_type="factored", bias_scale=0.1)
        return GatedCSSM(channels=C, **kw), p, orc.gated_forward, kw
    if name == "gdn":
        kw = dict(delta_key_dim=4, kernel_size=ks, rope_mode="mrope", gate_type="factored",
                  short_conv_size=4, qkv_conv_size=3)
        p = orc.init_gdn_params(2, C, H, W, delta_key_dim=4, kernel_size=ks, gate_type="factored",
                                short_conv_size=4, qkv_conv_size=3, bias_scale=0.1, perturb_rms=True)
        return GatedDeltaNetCSSM(channels=C, **kw), p, orc.gdn_forward, kw
    if name == "additive1":
        kw = dict(kernel_size=ks, rope_mode="spatiotemporal", gate_type="dense")
        p = orc.init_additive1_params(3, C, H, W, kernel_size=ks, gate_type="dense", bias_scale=0.1)
        return AdditiveCSSM(channels=C, single_state=True, **kw), p, orc.additive1_forward, kw
    if name == "deltanet":
        gt = "channel"
        kw = dict(kernel_size=ks, rope_mode="spatiotemporal", gate_type=gt)
        p = orc.init_deltanet_params(4, C, H, W, kernel_size=ks, gate_type=gt, bias_scale=0.1)
        p["output_proj"]["bias"][:] = 0
        return DeltaNetCSSM(channels=C, **kw), p, orc.deltanet_forward, kw
    p = {"kernel": (0.3 * rng.standard_normal((C, ks, ks))).astype(np.float32),
         "out_proj": {"kernel": (rng.standard_normal((C, C)) / np.sqrt(C)).astype(np.float32),
                      "bias": (0.1 * rng.standard_normal(C)).astype(np.float32)}}
    return NoGateCSSM(channels=C, kernel_size=ks), p, orc.nogate_forward, dict(kernel_size=ks)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("name", ["gated", "gdn", "additive1", "deltanet", "nogate"])
def test_special_inputs(name, shape):
    rng = np.random.default_rng(sum(map(ord, name)) * 1000 + shape[2] * shape[4])      # fixed per case
    mod, p, fwd, kw = _block(name, shape, rng)
    bound = mod.bind({"params": p})
    for kind in KINDS:
        x = _input(kind, shape, rng)
        ref = fwd(p, x, **kw)
        y = bound(torch.from_numpy(x).cuda()).cpu().numpy()
        assert np.isfinite(y).all(), kind
        assert orc.rel_l2(y, ref) <= TOL, kind
