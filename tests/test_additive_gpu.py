"""GPU parity of the single-state AdditiveCSSM block through the C ABI against the NumPy oracle.
Tolerance: rel-L2 <= 1e-4 in fp32."""
import os

import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from cssm_b200 import AdditiveCSSM

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _run(case, gate_type, rope, scan_mode="associative", seed=0):
    B, T, H, W, C, ks = case
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_additive1_params(seed + 1, C, H, W, kernel_size=ks, gate_type=gate_type,
                                  bias_scale=0.1)
    ref = orc.additive1_forward(p, x, kernel_size=ks, gate_type=gate_type, rope_mode=rope,
                                scan_mode=scan_mode)
    mod = AdditiveCSSM(channels=C, kernel_size=ks, single_state=True, gate_type=gate_type,
                       rope_mode=rope, scan_mode=scan_mode)
    y = mod.apply({"params": p}, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.isfinite(y).all()
    return orc.rel_l2(y, ref)


@pytest.mark.parametrize("case,gate_type,rope", [
    ((2, 5, 64, 64, 64, 11), "factored", "spatiotemporal"),   # 64x64 radix kernel, tensor-core GEMMs
    ((2, 4, 64, 64, 8, 11), "dense", "none"),                 # 64x64, CUDA-core GEMMs
    ((3, 6, 32, 32, 8, 11), "dense", "mrope"),                # 32x32 radix kernel
    ((2, 8, 32, 32, 64, 5), "factored", "none"),
    ((2, 3, 14, 10, 12, 3), "factored", "spatial_only"),      # small-plane kernel, ragged plane
    ((2, 3, 20, 18, 8, 7), "dense", "temporal"),              # generic kernel
    ((1, 1, 7, 7, 4, 11), "dense", "none"),                   # T = 1, kernel larger than the plane
    # per-channel decay, per-pixel 1x1-conv input / output gates ('channel') on all four kernels
    ((2, 4, 64, 64, 64, 11), "channel", "spatiotemporal"),
    ((1, 3, 64, 64, 8, 5), "channel", "none"),
    ((2, 5, 32, 32, 8, 11), "channel", "mrope"),
    ((2, 3, 14, 10, 12, 3), "channel", "temporal"),
    ((2, 3, 20, 18, 8, 7), "channel", "none"),
], ids=lambda c: "x".join(map(str, c)) if isinstance(c, tuple) else str(c))
def test_block_parity(case, gate_type, rope):
    assert _run(case, gate_type, rope) <= TOL


@pytest.mark.parametrize("scan_mode", ["ssd", "quadratic", "pallas"])
def test_linear_scan_modes(scan_mode):
    """The reference's other scan modes evaluate the same recurrence without the 1e-7 floors."""
    assert _run((2, 6, 32, 32, 8, 5), "factored", "spatiotemporal", scan_mode=scan_mode) <= TOL
    assert _run((1, 4, 64, 64, 8, 5), "dense", "none", scan_mode=scan_mode, seed=3) <= TOL


def test_state_decays_through_the_gated_kernel():
    """x_t = 0 for t > 0: the later frames are the first frame's state pushed through
    d_X,t * K_hat, so they are non-zero and must match the oracle frame by frame."""
    B, T, H, W, C, ks = 1, 4, 32, 32, 4, 5
    rng = np.random.default_rng(5)
    x = np.zeros((B, T, H, W, C), np.float32)
    x[:, 0] = rng.standard_normal((B, H, W, C))
    p = orc.init_additive1_params(6, C, H, W, kernel_size=ks, gate_type="dense", bias_scale=0.1)
    p["kernel"] = (0.5 * rng.standard_normal(p["kernel"].shape)).astype(np.float32)
    p["x_proj"]["bias"][:] = 0
    ref = orc.additive1_forward(p, x, kernel_size=ks)
    mod = AdditiveCSSM(channels=C, kernel_size=ks, single_state=True)
    y = mod.apply({"params": p}, torch.from_numpy(x).cuda()).cpu().numpy()
    for t in range(T):
        assert np.abs(ref[:, t]).max() > 1e-4
        assert orc.rel_l2(y[:, t], ref[:, t]) <= TOL


def test_out_argument_and_plan_reuse():
    B, T, H, W, C, ks = 2, 3, 32, 32, 8, 5
    x = torch.from_numpy(np.random.default_rng(7).standard_normal((B, T, H, W, C)).astype(np.float32)).cuda()
    mod = AdditiveCSSM(channels=C, kernel_size=ks, single_state=True, gate_type="factored")
    v = mod.init(8, tuple(x.shape), bias_scale=0.1)
    bound = mod.bind(v)
    y1 = bound(x)
    out = torch.empty_like(x)
    y2 = bound(x, out=out)
    assert y2.data_ptr() == out.data_ptr()
    assert torch.equal(y1, y2)
    assert len(bound._plans) == 1


def test_golden_fixture_on_gpu():
    """The committed fixture (tests/golden/additive1_small.npz, written by make_golden.py)."""
    from tests.golden import make_golden as mg
    g = np.load(os.path.join(os.path.dirname(mg.__file__), "additive1_small.npz"))
    _, p, kw = mg.additive1_case()
    mod = AdditiveCSSM(channels=g["x"].shape[-1], single_state=True, kernel_size=kw["kernel_size"],
                       gate_type=kw["gate_type"], rope_mode=kw["rope_mode"])
    y = mod.apply({"params": p}, torch.from_numpy(g["x"]).cuda()).cpu().numpy()
    assert orc.rel_l2(y, g["y"]) <= TOL
