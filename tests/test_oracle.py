"""CPU tests of the oracle: its two tiers against each other, the reference's scan-operator
test distributions against a sequential ground truth, structural invariants, the golden
vectors, and the timed torch-CPU restatement against the NumPy oracle."""
import os

import numpy as np
import pytest

from oracle import cssm_oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _scan_inputs(seed, shape, mag_lo=0.1):
    """|A| in [mag_lo, 0.95], uniform phase, U ~ N(0, .5^2) + i N(0, .5^2): the distributions
    of the reference's scan tests (tests/test_complex32.py:81-93, tests/test_ssd.py:77-87)."""
    rng = np.random.default_rng(seed)
    A = rng.uniform(mag_lo, 0.95, shape) * np.exp(1j * rng.uniform(-np.pi, np.pi, shape))
    U = 0.5 * rng.standard_normal(shape) + 0.5j * rng.standard_normal(shape)
    return A.astype(np.complex64), U.astype(np.complex64)


def _sequential(A, U):
    """benchmarks/bench_scan_modes.py:194-203."""
    h = np.zeros_like(A[:, 0], dtype=np.complex128)
    out = []
    for t in range(A.shape[1]):
        h = A[:, t].astype(np.complex128) * h + U[:, t]
        out.append(h)
    return np.stack(out, axis=1)


@pytest.mark.parametrize("T", [8, 16, 32])
def test_goom_scalar_scan_matches_sequential(T):
    A, U = _scan_inputs(T, (2, T, 4, 8, 5))
    got = orc.goom_scalar_scan(A, U)
    ref = _sequential(A, U)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 5e-6


@pytest.mark.parametrize("d", [2, 3, 4])
def test_goom_matrix_scan_matches_sequential(d):
    rng = np.random.default_rng(d)
    shape = (2, 8, 3, 4, 3)
    M = (0.4 * (rng.standard_normal(shape + (d, d)) + 1j * rng.standard_normal(shape + (d, d)))
         ).astype(np.complex64)
    U = (0.5 * (rng.standard_normal(shape + (d,)) + 1j * rng.standard_normal(shape + (d,)))
         ).astype(np.complex64)
    got = orc.goom_matrix_scan(M, U)
    u = np.zeros(shape[:1] + shape[2:] + (d,), np.complex128)
    ref = []
    for t in range(shape[1]):
        u = np.einsum("...ij,...j->...i", M[:, t].astype(np.complex128), u) + U[:, t]
        ref.append(u)
    ref = np.stack(ref, axis=1)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-5


def test_goom_floor_semantics():
    z = np.array([0.0, 5e-8, -5e-8j, 2e-7, -1.0], dtype=np.complex128)
    f = orc.goom_floor(z)
    assert f[0] == 1e-7 and f[1] == 1e-7 and f[2] == 1e-7
    assert f[3] == 2e-7 and f[4] == -1.0


GATED_CASES = [
    dict(B=2, T=4, H=8, W=8, C=8, ks=5, gt="dense", rope="spatiotemporal"),
    dict(B=1, T=8, H=16, W=16, C=4, ks=11, gt="factored", rope="mrope"),
    dict(B=2, T=1, H=7, W=7, C=12, ks=1, gt="factored", rope="none"),
    dict(B=1, T=32, H=8, W=8, C=4, ks=3, gt="dense", rope="temporal"),
]


@pytest.mark.parametrize("c", GATED_CASES, ids=lambda c: f"{c['H']}x{c['W']}T{c['T']}{c['gt']}")
def test_gated_tiers_agree(c):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((c["B"], c["T"], c["H"], c["W"], c["C"])).astype(np.float32)
    p = orc.init_gated_params(1, c["C"], c["H"], c["W"], kernel_size=c["ks"], gate_type=c["gt"],
                              bias_scale=0.1)
    kw = dict(kernel_size=c["ks"], rope_mode=c["rope"], gate_type=c["gt"])
    exact = orc.gated_forward(p, x, **kw)
    literal = orc.gated_forward(p, x, dtype=np.float32, scan="goom", **kw)
    assert orc.rel_l2(literal, exact) < 5e-6


@pytest.mark.parametrize("gt", ["factored", "dense"])
def test_gdn_tiers_agree(gt):
    rng = np.random.default_rng(0)
    B, T, H, W, C = 2, 4, 8, 8, 16
    x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_gdn_params(1, C, H, W, kernel_size=5, gate_type=gt, qkv_conv_size=5,
                            bias_scale=0.1, perturb_rms=True)
    kw = dict(kernel_size=5, rope_mode="mrope", gate_type=gt, qkv_conv_size=5)
    exact = orc.gdn_forward(p, x, **kw)
    literal = orc.gdn_forward(p, x, dtype=np.float32, scan="goom", **kw)
    assert orc.rel_l2(literal, exact) < 2e-5


def test_t1_output_independent_of_kernel():
    """h_1 = U_1: at T=1 the spectral kernel has no effect (cssm.py:570-572)."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 1, 8, 8, 8)).astype(np.float32)
    p = orc.init_gated_params(1, 8, 8, 8, kernel_size=3)
    y1 = orc.gated_forward(p, x, kernel_size=3)
    p2 = dict(p)
    p2["kernel"] = p["kernel"] * 7.0 + 1.0
    y2 = orc.gated_forward(p2, x, kernel_size=3)
    assert orc.rel_l2(y1, y2) < 1e-12


def test_kernel_size_one_gives_flat_spectrum():
    """ks=1 is a single centred tap: |K_hat| is constant over bins (linear phase only)."""
    k = np.random.default_rng(0).standard_normal((4, 1, 1)).astype(np.float32)
    K = orc.spectral_kernel(k, 16, 16)
    mag = np.abs(K)
    assert np.allclose(mag, mag[:, :1, :1], rtol=1e-12)
    assert (mag < 0.999).all()


def test_circular_shift_equivariance_without_convs_and_rope():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((1, 3, 8, 8, 4)).astype(np.float32)
    p = orc.init_gated_params(1, 4, 8, 8, kernel_size=3, short_conv_size=0,
                              short_conv_spatial_size=0, bias_scale=0.1)
    kw = dict(kernel_size=3, short_conv_size=0, short_conv_spatial_size=0)
    # the gates are indexed by frequency, so a spatial shift of the input shifts the output
    y = orc.gated_forward(p, x, **kw)
    ys = orc.gated_forward(p, np.roll(x, (2, 3), axis=(2, 3)), **kw)
    assert orc.rel_l2(ys, np.roll(y, (2, 3), axis=(2, 3))) < 1e-10


def test_irfft2_ignores_imag_of_dc_and_nyquist_columns():
    rng = np.random.default_rng(4)
    Y = rng.standard_normal((8, 5)) + 1j * rng.standard_normal((8, 5))
    a = np.fft.irfft2(Y, s=(8, 8))
    col = np.fft.ifft(Y, axis=0)
    col[:, 0] = col[:, 0].real
    col[:, 4] = col[:, 4].real
    b = np.fft.irfft(col, n=8, axis=1)
    assert np.abs(a - b).max() < 1e-14


def test_rope_modes_pair_rotation_is_orthogonal():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 3, 4, 5, 16))
    for mode in ("spatiotemporal", "temporal", "spatial_only", "mrope"):
        y = orc.apply_rope(x, mode)
        assert np.allclose((x ** 2).sum(-1), (y ** 2).sum(-1))
        assert np.allclose(y[:, 0, 0, 0], x[:, 0, 0, 0])      # angle 0 at the origin
    ft, fh, fw = orc.rope_axis_freqs(64, "spatiotemporal")
    assert (ft[:10] > 0).all() and (ft[10:] == 0).all()
    assert (fh[:11] > 0).all() and (fh[11:] == 0).all() and (fw[:11] > 0).all()
    ft, fh, fw = orc.rope_axis_freqs(64, "mrope")
    assert ((ft > 0).astype(int) + (fh > 0) + (fw > 0) == 1).all()   # one axis per pair


def test_golden_vectors():
    path = os.path.join(GOLDEN, "gated_small.npz")
    g = np.load(path)
    from tests.golden.make_golden import gated_case
    x, p, kw = gated_case()
    assert np.array_equal(x, g["x"])
    y = orc.gated_forward(p, x, **kw)
    assert orc.rel_l2(y, g["y"]) < 1e-12
    g2 = np.load(os.path.join(GOLDEN, "gdn_small.npz"))
    from tests.golden.make_golden import gdn_case
    x, p, kw = gdn_case()
    y = orc.gdn_forward(p, x, **kw)
    assert orc.rel_l2(y, g2["y"]) < 1e-12


def test_torch_cpu_restatement_matches_numpy_oracle():
    import torch
    from oracle import cssm_torch_cpu as tc
    rng = np.random.default_rng(0)
    B, T, H, W, C = 2, 3, 16, 16, 8
    x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
    for gt, rope in (("factored", "spatiotemporal"), ("dense", "mrope")):
        p = orc.init_gated_params(1, C, H, W, kernel_size=11, gate_type=gt, bias_scale=0.1)
        y = orc.gated_forward(p, x, kernel_size=11, rope_mode=rope, gate_type=gt)
        yt = tc.gated_forward_torch(p, torch.from_numpy(x), kernel_size=11, rope_mode=rope,
                                    gate_type=gt).numpy()
        assert orc.rel_l2(yt, y) < 1e-5


def test_additive1_oracle_scan_forms_agree():
    """Single-state AdditiveCSSM: the direct recurrence with the floors, the literal complex64
    log-space scan and the floor-free linear recurrence (ssd / quadratic / pallas modes) agree to
    fp32 rounding; with the gates forced to constants the block is the ungated recurrence scaled."""
    rng = np.random.default_rng(9)
    B, T, H, W, C, ks = 2, 5, 8, 6, 4, 3
    x = rng.standard_normal((B, T, H, W, C))
    for gt in ("dense", "factored"):
        p = orc.init_additive1_params(3, C, H, W, kernel_size=ks, gate_type=gt, bias_scale=0.1)
        a = orc.additive1_forward(p, x, kernel_size=ks, gate_type=gt, rope_mode="mrope")
        b = orc.additive1_forward(p, x, kernel_size=ks, gate_type=gt, rope_mode="mrope", scan="goom")
        c = orc.additive1_forward(p, x, kernel_size=ks, gate_type=gt, rope_mode="mrope", scan_mode="ssd")
        assert orc.rel_l2(b, a) < 5e-6
        assert orc.rel_l2(c, a) < 1e-6
    # zero gate weights: every gate is sigmoid(0) = 0.5 (d_X = 0.545), identity projections
    p = orc.init_additive1_params(4, C, H, W, kernel_size=ks, gate_type="dense")
    for n in ("d_X", "B_X", "C_gate"):
        p[n]["kernel"][:] = 0
    p["x_proj"] = {"kernel": np.eye(C), "bias": np.zeros(C)}
    p["output_proj"] = {"kernel": np.eye(C), "bias": np.zeros(C)}
    y = orc.additive1_forward(p, x, kernel_size=ks, scan_mode="pallas")
    K = orc.spectral_kernel(p["kernel"], H, W, 0.999)
    U = np.fft.rfft2(x.transpose(0, 1, 4, 2, 3), axes=(3, 4))
    h = np.zeros_like(U[:, 0])
    for t in range(T):
        h = 0.545 * K[None] * h + 0.5 * U[:, t]
        ref_t = np.fft.irfft2(0.5 * h, s=(H, W), axes=(2, 3)).transpose(0, 2, 3, 1)
        assert np.allclose(y[:, t], ref_t, atol=1e-12)


def test_deltanet_oracle_scan_forms_and_erasure():
    """DeltaNetCSSM: direct recurrence, literal log-space scan and floor-free recurrence agree;
    |A_t| < rho everywhere (the squash); with beta = 0 nothing is written, so the output is the
    output bias alone."""
    rng = np.random.default_rng(10)
    B, T, H, W, C, ks = 2, 5, 8, 6, 4, 3
    x = rng.standard_normal((B, T, H, W, C))
    for gt in ("dense", "factored"):
        p = orc.init_deltanet_params(5, C, H, W, kernel_size=ks, gate_type=gt, bias_scale=0.1)
        p["output_proj"]["bias"][:] = 0
        a = orc.deltanet_forward(p, x, kernel_size=ks, gate_type=gt, rope_mode="spatiotemporal")
        b = orc.deltanet_forward(p, x, kernel_size=ks, gate_type=gt, rope_mode="spatiotemporal", scan="goom")
        c = orc.deltanet_forward(p, x, kernel_size=ks, gate_type=gt, rope_mode="spatiotemporal", scan_mode="ssd")
        assert np.abs(a).max() > 1e-4
        assert orc.rel_l2(b, a) < 5e-6
        assert orc.rel_l2(c, a) < 1e-6
    p = orc.init_deltanet_params(6, C, H, W, kernel_size=ks, gate_type="dense", bias_scale=0.1)
    p["beta"]["kernel"][:] = 0
    p["beta"]["bias"][:] = -60.0                      # sigmoid -> 1e-26
    y = orc.deltanet_forward(p, x, kernel_size=ks, scan_mode="pallas")
    assert np.allclose(y, np.broadcast_to(p["output_proj"]["bias"], y.shape), atol=1e-12)


def test_nogate_oracle_is_a_circular_convolution_recurrence():
    """NoGateCSSM in the spatial domain: s_t = k (*) s_{t-1} + x_t with circular convolution by the
    inverse transform of the squashed kernel spectrum."""
    rng = np.random.default_rng(4)
    B, T, H, W, C, ks = 1, 3, 8, 8, 2, 3
    x = rng.standard_normal((B, T, H, W, C))
    p = {"kernel": 0.3 * rng.standard_normal((C, ks, ks)),
         "out_proj": {"kernel": np.eye(C), "bias": np.zeros(C)}}
    out = orc.nogate_forward(p, x, kernel_size=ks) + x           # undo the residual, identity out_proj
    K = orc.spectral_kernel(p["kernel"], H, W, 0.999)
    ksp = np.fft.irfft2(K, s=(H, W), axes=(1, 2))                 # (C,H,W) effective spatial kernel
    s = np.zeros((B, H, W, C))
    for t in range(T):
        nxt = np.zeros_like(s)
        for c in range(C):
            for dh in range(H):
                for dw in range(W):
                    nxt[..., c] += ksp[c, dh, dw] * np.roll(s[..., c], (dh, dw), axis=(1, 2))
        s = nxt + x[:, t]
        assert np.allclose(out[:, t], s, atol=1e-9)


def test_gdn_static_image_oracle_equals_general_path_last_frame():
    """With the bf16 carry switched off, the static-image fast path is the general path on the
    clip that repeats the image, read at the last frame (no short conv, no input gates, no RoPE)."""
    rng = np.random.default_rng(1)
    B, H, W, C, T = 2, 8, 8, 8, 4
    x = rng.standard_normal((B, H, W, C))
    p = orc.init_gdn_params(3, C, H, W, delta_key_dim=4, kernel_size=5, gate_type="factored",
                            short_conv_size=0, qkv_conv_size=3, use_input_gates=False,
                            bias_scale=0.1, perturb_rms=True)
    y64 = orc.gdn_static_forward(p, x, num_timesteps=T, kernel_size=5, qkv_conv_size=3, carry="fp64")
    yg = orc.gdn_forward(p, np.repeat(x[:, None], T, axis=1), delta_key_dim=4, kernel_size=5,
                         rope_mode="none", gate_type="factored", short_conv_size=0, qkv_conv_size=3,
                         use_input_gates=False)
    assert orc.rel_l2(y64, yg[:, -1]) <= 1e-12
    y = orc.gdn_static_forward(p, x, num_timesteps=T, kernel_size=5, qkv_conv_size=3)
    assert 1e-5 < orc.rel_l2(y, y64) < 2e-2          # what the bf16 carry costs


def test_bf16_round_matches_torch():
    import torch
    a = (np.random.default_rng(0).standard_normal(4096) * 3).astype(np.float32)
    ref = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(orc.bf16_round(a), ref)


def test_golden_vectors_of_the_widened_paths():
    """Committed fixtures of the SimpleCSSM model, NoGateCSSM and the GDN static-image path
    (tests/golden/make_golden.py) pin the oracle against drift."""
    from oracle import simple_oracle as so
    from tests.golden import make_golden as mg
    g = np.load(os.path.join(GOLDEN, "simple_small.npz"))
    x, p = mg.simple_case()
    assert np.array_equal(x, g["x"])
    y = so.simple_forward(p, x, seq_len=3, stem_layers=1, pool_type="max", block_kwargs=mg.SIMPLE_KW)
    assert orc.rel_l2(y, g["y"]) < 1e-12
    g = np.load(os.path.join(GOLDEN, "nogate_small.npz"))
    x, p, ks = mg.nogate_case()
    assert np.array_equal(x, g["x"])
    assert orc.rel_l2(orc.nogate_forward(p, x, kernel_size=ks), g["y"]) < 1e-12
    g = np.load(os.path.join(GOLDEN, "additive1_small.npz"))
    x, p, kw = mg.additive1_case()
    assert np.array_equal(x, g["x"])
    assert orc.rel_l2(orc.additive1_forward(p, x, **kw), g["y"]) < 1e-12
    g = np.load(os.path.join(GOLDEN, "deltanet_small.npz"))
    x, p, kw = mg.deltanet_case()
    assert np.array_equal(x, g["x"])
    assert orc.rel_l2(orc.deltanet_forward(p, x, **kw), g["y"]) < 1e-12
    g = np.load(os.path.join(GOLDEN, "gdn_static_small.npz"))
    x, p, kw = mg.gdn_static_case()
    assert np.array_equal(x, g["x"])
    assert orc.rel_l2(orc.gdn_static_forward(p, x, **kw), g["y"]) < 1e-12
