"""CPU checks of the SimpleCSSM model oracle: the NumPy restatement against independent
formulations of its pieces, and the torch-CPU restatement (the timed CPU baseline) against it."""
import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from oracle import cssm_torch_cpu as tc
from oracle import simple_oracle as so

GATED_KW = dict(kernel_size=5, rope_mode="spatiotemporal", gate_type="factored", short_conv_size=4,
                short_conv_spatial_size=3)
GDN_KW = dict(kernel_size=5, rope_mode="mrope", delta_key_dim=4, qkv_conv_size=3, gate_type="factored")


def test_stem_pieces_against_torch_functional():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 9, 11, 3))
    p = {"kernel": rng.standard_normal((3, 3, 3, 8)), "bias": rng.standard_normal(8)}
    ref = torch.nn.functional.conv2d(torch.from_numpy(x).permute(0, 3, 1, 2),
                                     torch.from_numpy(p["kernel"]).permute(3, 2, 0, 1),
                                     torch.from_numpy(p["bias"]), padding=1).permute(0, 2, 3, 1).numpy()
    assert np.allclose(so.conv2d_same(x, p), ref, atol=1e-12)
    y = rng.standard_normal((2, 9, 11, 8))
    pool = torch.nn.functional.max_pool2d(torch.from_numpy(y).permute(0, 3, 1, 2), 2, 2,
                                          ceil_mode=True).permute(0, 2, 3, 1).numpy()
    assert np.array_equal(so.max_pool_2x2_same(y), pool)          # odd sizes: -inf padding
    ln = {"scale": rng.standard_normal(8), "bias": rng.standard_normal(8)}
    refln = torch.nn.functional.layer_norm(torch.from_numpy(y), (8,), torch.from_numpy(ln["scale"]),
                                           torch.from_numpy(ln["bias"]), eps=1e-6).numpy()
    assert np.allclose(so.layer_norm(y, ln), refln, atol=1e-10)


def test_image_input_equals_repeated_clip():
    """A 4-D image batch gives the logits of the clip that repeats each image seq_len times
    (src/models/simple_cssm.py:238-241)."""
    rng = np.random.default_rng(1)
    x = rng.random((2, 16, 16, 1))
    p = so.init_simple_params(0, cin=1, embed_dim=8, H=8, W=8, stem_layers=1, block_kwargs=GATED_KW)
    a = so.simple_forward(p, x, seq_len=3, stem_layers=1, block_kwargs=GATED_KW)
    b = so.simple_forward(p, np.repeat(x[:, None], 3, axis=1), seq_len=99, stem_layers=1,
                          block_kwargs=GATED_KW)
    assert np.allclose(a, b, atol=1e-12)


@pytest.mark.parametrize("ct,kw,shape,stem_mode", [
    ("gated", GATED_KW, (2, 16, 16, 1), "default"),
    ("gdn", GDN_KW, (2, 17, 16, 2), "default"),
    ("gdn", dict(GDN_KW, qkv_conv_size=1, gate_type="dense"), (2, 4, 8, 8, 3), "pathtracker"),
])
def test_torch_cpu_model_matches_numpy_oracle(ct, kw, shape, stem_mode):
    H, W = (shape[-3], shape[-2]) if stem_mode == "pathtracker" else ((shape[-3] + 1) // 2, (shape[-2] + 1) // 2)
    p = so.init_simple_params(0, cin=shape[-1], embed_dim=8, H=H, W=W, cssm_type=ct,
                              stem_mode=stem_mode, stem_layers=1, block_kwargs=kw)
    x = np.random.default_rng(1).random(shape).astype(np.float32)
    ref = so.simple_forward(p, x, cssm_type=ct, seq_len=3, stem_mode=stem_mode, stem_layers=1,
                            pool_type="max", block_kwargs=kw)
    out = tc.simple_forward_torch(p, torch.from_numpy(x), cssm_type=ct, seq_len=3,
                                  stem_mode=stem_mode, stem_layers=1, pool_type="max",
                                  block_kwargs=kw).numpy()
    assert orc.rel_l2(out, ref) <= 2e-5


def test_gdn_torch_block_matches_numpy_oracle():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 8, 8, 8)).astype(np.float32)
    p = orc.init_gdn_params(3, 8, 8, 8, delta_key_dim=4, kernel_size=5, gate_type="factored",
                            qkv_conv_size=3, bias_scale=0.1, perturb_rms=True)
    kw = dict(delta_key_dim=4, kernel_size=5, rope_mode="mrope", gate_type="factored", qkv_conv_size=3)
    ref = orc.gdn_forward(p, x, **kw)
    out = tc.gdn_forward_torch(p, torch.from_numpy(x), **kw).numpy()
    assert orc.rel_l2(out, ref) <= 2e-5
