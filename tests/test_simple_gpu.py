"""GPU parity of the SimpleCSSM model path (stem, block + residual, last-frame readout) through
the C ABI against the NumPy oracle.  Tolerance: rel-L2 <= 1e-4 on features and logits (fp32)."""
import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from oracle import simple_oracle as so
from cssm_b200 import SimpleCSSM

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _model(cssm_type, E, ks, pos, stem_mode, stem_layers, pool, rnorm, **extra):
    return SimpleCSSM(num_classes=extra.pop("num_classes", 2), embed_dim=E, cssm_type=cssm_type,
                      kernel_size=ks, pos_embed=pos, stem_mode=stem_mode, stem_layers=stem_layers,
                      pool_type=pool, readout_norm=rnorm, gate_type=extra.pop("gate_type", "factored"),
                      **extra)


def _block_kwargs(m):
    rope = m.pos_embed if m.pos_embed != "none" else "none"
    if m.cssm_type == "gated":
        return dict(kernel_size=m.kernel_size, rope_mode=rope, gate_type=m.gate_type,
                    short_conv_size=m.short_conv_size,
                    short_conv_spatial_size=m.short_conv_spatial_size)
    if m.cssm_type == "no_gate":
        return dict(kernel_size=m.kernel_size)
    if m.cssm_type in ("add_kqv_1", "deltanet"):
        return dict(kernel_size=m.kernel_size, rope_mode=rope, gate_type=m.gate_type,
                    scan_mode=m.scan_mode)
    return dict(delta_key_dim=m.delta_key_dim, kernel_size=m.kernel_size, rope_mode=rope,
                gate_type=m.gate_type, short_conv_size=m.short_conv_size,
                qkv_conv_size=m.qkv_conv_size)


CASES = [
    # cssm_type, E, ks, pos_embed, stem_mode, stem_layers, pool, readout_norm, x shape, extra
    ("gated", 8, 5, "spatiotemporal", "default", 1, "max", "pre", (3, 16, 16, 1), dict(seq_len=3)),
    ("gated", 8, 3, "none", "default", 2, "mean", "post", (2, 20, 20, 3), dict(seq_len=2)),
    ("gated", 64, 11, "spatiotemporal", "default", 1, "max", "pre", (2, 128, 128, 1), dict(seq_len=4)),
    # two stem layers with 16 / 64 channels: the second layer runs the weight-reusing kernel
    ("gated", 16, 3, "none", "default", 2, "max", "pre", (2, 22, 26, 1), dict(seq_len=2)),
    ("gated", 16, 3, "none", "default", 2, "max", "pre", (40, 90, 94, 1), dict(seq_len=1)),   # a full wave of windows
    ("gated", 64, 1, "spatiotemporal", "default", 2, "mean", "pre", (2, 128, 128, 1),
     dict(seq_len=1, gate_type="dense")),
    ("gated", 16, 5, "mrope", "default", 1, "mean", "pre", (2, 3, 14, 18, 2), dict()),        # clips, odd pool
    ("gdn", 8, 5, "mrope", "pathtracker", 1, "mean", "pre", (2, 4, 8, 8, 3), dict(delta_key_dim=4)),
    ("gdn", 64, 11, "spatiotemporal", "pathtracker", 1, "max", "pre", (2, 5, 32, 32, 3),
     dict(delta_key_dim=4, num_classes=3)),
    ("gdn", 16, 11, "mrope", "default", 1, "max", "pre", (2, 64, 64, 1),
     dict(delta_key_dim=4, qkv_conv_size=5, seq_len=3)),                                     # image input, dwconv
    ("gdn", 8, 3, "none", "default", 1, "mean", "pre", (2, 16, 16, 1),
     dict(delta_key_dim=4, qkv_conv_size=1, seq_len=3)),                                     # image input, no dwconv
    # the scalar-scan blocks under their registry names: image input (features repeated over T) and clips
    ("no_gate", 8, 5, "none", "default", 1, "max", "pre", (2, 16, 16, 1), dict(seq_len=3)),
    ("no_gate", 16, 11, "none", "pathtracker", 1, "mean", "pre", (2, 4, 32, 32, 3), dict()),
    ("add_kqv_1", 8, 5, "spatiotemporal", "default", 1, "max", "pre", (2, 16, 16, 1), dict(seq_len=3)),
    ("add_kqv_1", 64, 11, "mrope", "default", 1, "max", "pre", (2, 128, 128, 1),
     dict(seq_len=4, gate_type="dense", scan_mode="ssd")),
    ("add_kqv_1", 16, 3, "none", "pathtracker", 1, "mean", "post", (2, 5, 32, 32, 3), dict()),
    ("deltanet", 8, 5, "spatiotemporal", "default", 1, "max", "pre", (2, 16, 16, 1),
     dict(seq_len=3, gate_type="channel")),
    ("deltanet", 16, 11, "mrope", "default", 1, "mean", "pre", (2, 128, 128, 1), dict(seq_len=3)),
    ("deltanet", 8, 3, "none", "pathtracker", 1, "max", "pre", (2, 4, 12, 10, 3), dict(gate_type="dense")),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[0]}-E{c[1]}-{c[4]}{c[5]}-{'x'.join(map(str, c[8]))}")
def test_model_parity(case):
    cssm_type, E, ks, pos, stem_mode, layers, pool, rnorm, xshape, extra = case
    m = _model(cssm_type, E, ks, pos, stem_mode, layers, pool, rnorm, **dict(extra))
    rng = np.random.default_rng(3)
    x = rng.random(xshape).astype(np.float32)
    H, W = m.feature_hw(xshape[-3], xshape[-2])
    bkw = _block_kwargs(m)
    p = so.init_simple_params(5, cin=xshape[-1], embed_dim=E, H=H, W=W, num_classes=m.num_classes,
                              cssm_type=cssm_type, stem_mode=stem_mode, stem_layers=layers,
                              bias_scale=0.1, block_kwargs=bkw)
    ref, inter = so.simple_forward(p, x, cssm_type=cssm_type, seq_len=m.seq_len, stem_mode=stem_mode,
                                   stem_layers=layers, pool_type=pool, readout_norm=rnorm,
                                   block_kwargs=bkw, return_intermediates=True)
    bound = m.bind({"params": p})
    xd = torch.from_numpy(x).cuda()
    feat = bound.stem(xd).cpu().numpy()
    ref_feat = inter["stem"][:, 0] if len(xshape) == 4 else inter["stem"]
    assert orc.rel_l2(feat, ref_feat) <= TOL
    logits = bound(xd).cpu().numpy()
    assert np.isfinite(logits).all()
    assert orc.rel_l2(logits, ref) <= TOL
    # the last-frame-only evaluation of the block gives the same logits
    logits_last = bound(xd, last_frame_only=True).cpu().numpy()
    assert orc.rel_l2(logits_last, logits) <= 1e-5
    # host-buffer entry point
    lh = bound.forward_host(torch.from_numpy(x).pin_memory()).numpy()
    assert np.array_equal(lh, logits)


@pytest.mark.parametrize("cssm_type", ["gated", "gdn", "no_gate", "add_kqv_1", "deltanet"])
def test_sparse_stroke_images(cssm_type):
    """The benchmark's stroke images (94 % background): most stem pixels have all channels equal,
    which LayerNorm must map to exactly zero; every mixer follows the stem."""
    from cssm_b200 import synth
    extra = dict(delta_key_dim=4, qkv_conv_size=3) if cssm_type == "gdn" else {}
    m = _model(cssm_type, 16, 5, "spatiotemporal" if cssm_type != "no_gate" else "none", "default", 1,
               "max", "pre", seq_len=3, **extra)
    x = synth.stroke_batch(3, seed0=4000)
    H, W = m.feature_hw(128, 128)
    bkw = _block_kwargs(m)
    p = so.init_simple_params(9, cin=1, embed_dim=16, H=H, W=W, num_classes=2, cssm_type=cssm_type,
                              stem_mode="default", stem_layers=1, bias_scale=0.0, block_kwargs=bkw)
    ref, inter = so.simple_forward(p, x, cssm_type=cssm_type, seq_len=3, stem_mode="default",
                                   stem_layers=1, pool_type="max", readout_norm="pre",
                                   block_kwargs=bkw, return_intermediates=True)
    bound = m.bind({"params": p})
    xd = torch.from_numpy(x).cuda()
    feat = bound.stem(xd).cpu().numpy()
    assert orc.rel_l2(feat, inter["stem"][:, 0]) <= 1e-5
    background = np.abs(inter["stem"][:, 0]).max(-1) == 0          # exact zeros in the oracle
    assert background.mean() > 0.5
    assert np.abs(feat[background]).max() == 0.0
    assert orc.rel_l2(bound(xd).cpu().numpy(), ref) <= TOL


def test_unsupported_fields_raise():
    with pytest.raises(NotImplementedError):
        SimpleCSSM(cssm_type="gated", depth=2).bind({"params": {}})
    with pytest.raises(NotImplementedError):
        SimpleCSSM(cssm_type="hgru_bi").bind({"params": {}})
    with pytest.raises(NotImplementedError):
        SimpleCSSM(cssm_type="add_kqv_1", learned_init=True).bind({"params": {}})
    with pytest.raises(NotImplementedError):
        SimpleCSSM(cssm_type="deltanet", gate_type="scalar").bind({"params": {}})
    with pytest.raises(NotImplementedError):
        SimpleCSSM(cssm_type="gated", embed_dim=128).bind({"params": {}})


def test_golden_fixture_on_gpu():
    """The committed model fixture (tests/golden/simple_small.npz, written by make_golden.py)."""
    import os
    from tests.golden import make_golden as mg
    g = np.load(os.path.join(os.path.dirname(mg.__file__), "simple_small.npz"))
    _, p = mg.simple_case()
    m = SimpleCSSM(cssm_type="gated", embed_dim=8, kernel_size=5, pos_embed="spatiotemporal",
                   gate_type="factored", seq_len=3, stem_layers=1, pool_type="max")
    logits = m.apply({"params": p}, torch.from_numpy(g["x"]).cuda()).cpu().numpy()
    assert orc.rel_l2(logits, g["y"]) <= TOL


def test_streaming_host_entry_prefetches_the_next_batch():
    """forward_host_pipelined: prefetched, cold and dropped-prefetch batches all give the device
    entry point's logits, for image and clip inputs."""
    for shape, extra in (((4, 32, 32, 1), dict(seq_len=3)), ((2, 4, 16, 16, 3), dict(stem_mode="pathtracker"))):
        m = _model("gated", 8, 5, "spatiotemporal", extra.pop("stem_mode", "default"), 1, "max", "pre", **extra)
        rng = np.random.default_rng(3)
        xs = [torch.from_numpy(rng.random(shape).astype(np.float32)).pin_memory() for _ in range(3)]
        v = m.init(0, shape)
        bound = m.bind(v)
        want = [bound(x.cuda()).cpu() for x in xs]
        lh = torch.empty_like(want[0]).pin_memory()
        bound.forward_host_pipelined(xs[0], xs[1], lh)      # cold, prefetches xs[1]
        assert torch.equal(lh, want[0])
        bound.forward_host_pipelined(xs[1], xs[2], lh)      # prefetched
        assert torch.equal(lh, want[1])
        bound.forward_host_pipelined(xs[0], None, lh)       # the prefetch of xs[2] is dropped
        assert torch.equal(lh, want[0])
        bound.forward_host_pipelined(xs[2], xs[2], lh, last_frame_only=True)
        assert orc.rel_l2(lh.numpy(), want[2].numpy()) <= 1e-5
        bound.close()
