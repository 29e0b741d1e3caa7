"""Case table shared by the fixture generator (make_reference_golden.py, which runs the
reference's own model files) and by the tests that read the fixtures.

Every case names: the reference class and its constructor arguments; the oracle function
(`oracle/cssm_oracle.py` / `simple_oracle.py` / `shvit_oracle.py`) with its keyword arguments;
the module mirror in `cssm_b200` with its arguments (None where the library has no mirror for
the case); and a seeded input.  Inputs are regenerated from the seed, parameters and reference
outputs are read from `tests/golden/ref/<name>.npz`."""
from __future__ import annotations

import os
import zlib

import numpy as np

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref")
MAX_STORED = 32768          # outputs with more elements are stored at this many seeded positions


def make_input(case):
    rng = np.random.default_rng(case["seed"])
    shape = tuple(case["shape"])
    kind = case.get("input", "normal")
    if kind == "normal":
        x = rng.standard_normal(shape)
    elif kind == "uniform":
        x = rng.random(shape)
    elif kind == "sparse":                      # exact zeros on ~94 % of the pixels (stroke-like)
        x = rng.random(shape) * (rng.random(shape[:-1] + (1,)) < 0.06)
    else:
        raise ValueError(kind)
    return x.astype(np.float32)


def stored_positions(name, size):
    if size <= MAX_STORED:
        return None
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    return np.sort(rng.choice(size, MAX_STORED, replace=False))


def flatten(tree, prefix=""):
    out = {}
    for k, v in tree.items():
        if isinstance(v, dict):
            out.update(flatten(v, prefix + k + "/"))
        else:
            out[prefix + k] = np.asarray(v)
    return out


def unflatten(flat):
    tree = {}
    for key, v in flat.items():
        node = tree
        parts = key.split("/")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = v
    return tree


def seeded_params(case):
    """Parameter trees that are regenerated from a seed instead of stored (the full-size model)."""
    from oracle import shvit_oracle as sv
    kind, seed, kw = case["seeded_params"]
    assert kind == "shvit"
    return sv.init_shvit_params(seed, **kw)


def load(name):
    """-> (params tree (float32), batch_stats tree or None, stored reference values (float64),
    positions or None)."""
    with np.load(os.path.join(REF_DIR, name + ".npz")) as z:
        if "seeded_params" in BY_NAME[name]:
            params, stats = seeded_params(BY_NAME[name])
        else:
            params = unflatten({k[2:]: z[k] for k in z.files if k.startswith("p:")})
            stats = unflatten({k[2:]: z[k] for k in z.files if k.startswith("s:")}) or None
        pos = z["positions"] if "positions" in z.files else None
        return params, stats, z["y"], pos


def pick(y, pos):
    y = np.asarray(y, np.float64).ravel()
    return y if pos is None else y[pos]


def rel_err(got, ref):
    """||got - ref|| over the norm of ref's variation about its per-channel mean (a large constant
    bias in the last layer must not hide an error in the signal)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref - ref.mean()), 1e-30))


def _gated(name, shape, seed, input="normal", **kw):
    ref = dict(channels=shape[-1], **kw)
    okw = dict(kw)
    if "gate_activation" in okw:
        okw["gate_activation_kind"] = okw.pop("gate_activation")
    okw.setdefault("kernel_size", 15)
    return dict(name=name, family="gated", ref_class="GatedCSSM", ref_kwargs=ref,
                oracle="gated_forward", oracle_kwargs=okw, mirror="GatedCSSM", mirror_kwargs=ref,
                shape=shape, seed=seed, input=input)


def _gdn(name, shape, seed, mirror=True, **kw):
    ref = dict(channels=shape[-1], delta_key_dim=4, **kw)
    okw = dict(delta_key_dim=4, **kw)
    return dict(name=name, family="gdn", ref_class="GatedDeltaNetCSSM", ref_kwargs=ref,
                oracle="gdn_forward", oracle_kwargs=okw,
                mirror="GatedDeltaNetCSSM" if mirror else None, mirror_kwargs=ref,
                shape=shape, seed=seed)


def _gdn_static(name, shape, seed, T, **kw):
    ref = dict(channels=shape[-1], delta_key_dim=4, static_image_fast_path=True, num_timesteps=T,
               short_conv_size=0, use_input_gates=False, rope_mode="none", **kw)
    okw = dict(num_timesteps=T, delta_key_dim=4, **kw)
    return dict(name=name, family="gdn_static", ref_class="GatedDeltaNetCSSM", ref_kwargs=ref,
                oracle="gdn_static_forward", oracle_kwargs=okw, mirror="GatedDeltaNetCSSM",
                mirror_kwargs=ref, shape=shape, seed=seed, tol_oracle=2e-2, tol_gpu=2e-2)


def _nogate(name, shape, seed, **kw):
    ref = dict(channels=shape[-1], **kw)
    return dict(name=name, family="nogate", ref_class="NoGateCSSM", ref_kwargs=ref,
                oracle="nogate_forward", oracle_kwargs=dict(kw), mirror="NoGateCSSM",
                mirror_kwargs=ref, shape=shape, seed=seed, spectral_scale=6.0)


def _additive(name, shape, seed, **kw):
    ref = dict(channels=shape[-1], single_state=True, **kw)
    return dict(name=name, family="additive1", ref_class="AdditiveCSSM", ref_kwargs=ref,
                oracle="additive1_forward", oracle_kwargs=dict(kw), mirror="AdditiveCSSM",
                mirror_kwargs=ref, shape=shape, seed=seed)


def _deltanet(name, shape, seed, **kw):
    ref = dict(channels=shape[-1], **kw)
    return dict(name=name, family="deltanet", ref_class="DeltaNetCSSM", ref_kwargs=ref,
                oracle="deltanet_forward", oracle_kwargs=dict(kw), mirror="DeltaNetCSSM",
                mirror_kwargs=ref, shape=shape, seed=seed)


def _simple(name, shape, seed, block_kwargs, **kw):
    """SimpleCSSM: kw are SimpleCSSM fields (reference names)."""
    ref = dict(depth=1, frame_readout="last", norm_type="layer", act_type="softplus", **kw)
    return dict(name=name, family="simple", ref_class="SimpleCSSM", ref_kwargs=ref,
                oracle="simple_forward", block_kwargs=block_kwargs, mirror="SimpleCSSM",
                mirror_kwargs=ref, shape=shape, seed=seed, input="uniform", call_kwargs=dict(training=False))


def _shvit(name, shape, seed, seeded=None, mirror_dtype="bfloat16", **kw):
    """CSSMSHViT with gated mixers; kw are CSSMSHViT fields."""
    ref = dict(cssm_type="gated", **kw)
    okw = {k: v for k, v in kw.items() if k not in ("num_classes", "mlp_ratio", "drop_path_rate")}
    c = dict(name=name, family="shvit", ref_class="CSSMSHViT", ref_kwargs=ref,
             oracle="shvit_forward", oracle_kwargs=okw, mirror="CSSMSHViT",
             mirror_kwargs=dict(ref, dtype=mirror_dtype), shape=shape, seed=seed,
             call_kwargs=dict(training=False),
             tol_gpu=2e-2 if mirror_dtype == "bfloat16" else 1e-4)
    if seeded is not None:
        init_kw = {k: v for k, v in kw.items() if k in (
            "embed_dims", "depths", "use_cssm_stages", "kernel_sizes", "num_classes", "mlp_ratio",
            "gate_type", "short_conv_size", "short_conv_spatial_size", "use_pos_conv", "use_dwconv")}
        c["seeded_params"] = ("shvit", seeded, dict(in_hw=shape[1:3], **init_kw))
    return c


def _shvit_block(name, shape, seed, **kw):
    ref = dict(dim=shape[-1], cssm_type="gated", **kw)
    okw = dict(kw)
    return dict(name=name, family="shvit_block", ref_class="CSSMSHViTBlock", ref_kwargs=ref,
                oracle="cssm_block", oracle_kwargs=okw, mirror="CSSMSHViTBlock",
                mirror_kwargs=ref, shape=shape, seed=seed, tol_gpu=2e-2)


_S1 = dict(embed_dims=(64, 128, 256, 384), depths=(1, 2, 2, 1), num_classes=1000)

CASES = [
    # ---- GatedCSSM: the BASELINE block configurations at small batch / channel counts
    _gated("gated_cfg1_ks1_T1_dense", (2, 1, 32, 32, 8), 101, kernel_size=1, gate_type="dense",
           rope_mode="spatiotemporal"),
    _gated("gated_cfg2_ks11_T8_factored_64", (1, 8, 64, 64, 4), 102, kernel_size=11,
           gate_type="factored", rope_mode="spatiotemporal"),
    _gated("gated_cfg2_c64_T2_64", (1, 2, 64, 64, 64), 103, kernel_size=11, gate_type="factored",
           rope_mode="spatiotemporal"),
    _gated("gated_cfg2_sparse_32", (2, 4, 32, 32, 8), 104, input="sparse", kernel_size=11,
           gate_type="factored", rope_mode="spatiotemporal"),
    _gated("gated_cfg5_stage2_14", (3, 1, 14, 14, 16), 105, kernel_size=1, gate_type="factored",
           short_conv_spatial_size=0),
    _gated("gated_cfg5_stage3_7", (3, 1, 7, 7, 24), 106, kernel_size=1, gate_type="factored",
           short_conv_spatial_size=0),
    # ---- every RoPE mode (C/2 a multiple of 3 and not)
    _gated("gated_rope_mrope_c12", (2, 3, 8, 10, 12), 111, kernel_size=5, gate_type="factored",
           rope_mode="mrope"),
    _gated("gated_rope_mrope_c8", (2, 3, 8, 10, 8), 112, kernel_size=5, gate_type="factored",
           rope_mode="mrope"),
    _gated("gated_rope_spatiotemporal_c12", (2, 3, 8, 10, 12), 113, kernel_size=5,
           gate_type="dense", rope_mode="spatiotemporal"),
    _gated("gated_rope_temporal", (2, 5, 8, 8, 8), 114, kernel_size=3, gate_type="factored",
           rope_mode="temporal"),
    _gated("gated_rope_spatial_only", (2, 2, 10, 8, 8), 115, kernel_size=3, gate_type="factored",
           rope_mode="spatial_only", rope_base=100.0),
    # ---- gate activations, kernel larger than the plane, convs off, ragged plane
    _gated("gated_act_sigmoid", (2, 4, 8, 8, 8), 121, kernel_size=5, gate_type="dense",
           gate_activation="sigmoid"),
    _gated("gated_act_exp", (2, 4, 8, 8, 8), 122, kernel_size=5, gate_type="factored",
           gate_activation="exp"),
    _gated("gated_ks_gt_plane", (2, 3, 8, 8, 8), 123, kernel_size=11, gate_type="factored"),
    _gated("gated_no_short_convs", (2, 3, 16, 16, 8), 124, kernel_size=7, gate_type="factored",
           short_conv_size=0, short_conv_spatial_size=0, spectral_rho=0.9),
    _gated("gated_ragged_14x10_conv5", (2, 3, 14, 10, 8), 125, kernel_size=5, gate_type="dense",
           short_conv_spatial_size=5, short_conv_size=2, rope_mode="spatiotemporal"),
    _gated("gated_T32_32", (1, 32, 32, 32, 4), 126, kernel_size=11, gate_type="factored",
           rope_mode="spatiotemporal"),
    # ---- GatedDeltaNetCSSM (general path)
    _gdn("gdn_cfg3_ks11_qkv5_mrope_32", (1, 8, 32, 32, 8), 201, kernel_size=11, qkv_conv_size=5,
         rope_mode="mrope", gate_type="factored", output_norm="rms"),
    _gdn("gdn_cfg3_64", (1, 2, 64, 64, 8), 202, kernel_size=11, qkv_conv_size=5,
         rope_mode="mrope", gate_type="factored"),
    _gdn("gdn_cfg4_T8_32", (1, 8, 32, 32, 8), 203, kernel_size=11, gate_type="factored",
         rope_mode="spatiotemporal"),
    _gdn("gdn_dense_gates", (2, 3, 8, 8, 8), 204, kernel_size=5, gate_type="dense",
         rope_mode="none"),
    _gdn("gdn_no_l2_sigmoid_gate", (2, 3, 8, 10, 8), 205, kernel_size=5, gate_type="factored",
         use_spectral_l2_norm=False, output_gate_act="sigmoid", no_spectral_clamp=True),
    _gdn("gdn_no_input_gates_no_conv", (2, 3, 8, 8, 8), 206, kernel_size=3, gate_type="factored",
         use_input_gates=False, short_conv_size=0),
    _gdn("gdn_norm_none", (2, 2, 8, 8, 8), 207, kernel_size=5, gate_type="factored",
         output_norm="none", qkv_conv_size=3),
    _gdn("gdn_channel_gates", (2, 3, 8, 8, 8), 208, kernel_size=5, gate_type="channel",
         rope_mode="mrope"),
    _gdn("gdn_scalar_gates", (2, 3, 8, 8, 8), 209, kernel_size=5, gate_type="scalar"),
    # ---- GDN static-image fast path (bf16 carry)
    _gdn_static("gdn_static_T4_16", (2, 16, 16, 8), 251, 4, kernel_size=5, gate_type="factored"),
    _gdn_static("gdn_static_T8_32_qkv3", (1, 32, 32, 8), 252, 8, kernel_size=11,
                gate_type="factored", qkv_conv_size=3),
    # ---- scalar-scan relatives
    _nogate("nogate_ks3", (2, 4, 8, 8, 8), 301, kernel_size=3),
    _nogate("nogate_ks11_32", (1, 8, 32, 32, 4), 302, kernel_size=11),
    _additive("additive1_factored", (2, 4, 8, 8, 8), 311, kernel_size=5, gate_type="factored",
              rope_mode="spatiotemporal"),
    _additive("additive1_dense_mrope", (2, 4, 8, 10, 12), 312, kernel_size=5, gate_type="dense",
              rope_mode="mrope"),
    _additive("additive1_ssd", (1, 8, 8, 8, 8), 313, kernel_size=5, gate_type="dense",
              scan_mode="ssd"),
    _additive("additive1_quadratic", (1, 8, 8, 8, 8), 314, kernel_size=5, gate_type="dense",
              scan_mode="quadratic"),
    _additive("additive1_channel", (2, 4, 8, 10, 8), 315, kernel_size=5, gate_type="channel",
              rope_mode="mrope"),
    _additive("additive1_channel_32", (1, 3, 32, 32, 8), 316, kernel_size=11, gate_type="channel"),
    _additive("additive1_channel_64", (1, 2, 64, 64, 4), 317, kernel_size=11, gate_type="channel",
              rope_mode="spatiotemporal"),
    _deltanet("deltanet_channel", (2, 4, 8, 8, 8), 321, kernel_size=5, gate_type="channel",
              rope_mode="mrope"),
    _deltanet("deltanet_dense", (2, 4, 8, 8, 8), 322, kernel_size=5, gate_type="dense"),
    _deltanet("deltanet_factored_64", (1, 2, 64, 64, 4), 323, kernel_size=11,
              gate_type="factored", rope_mode="spatiotemporal"),
    # ---- SimpleCSSM around the blocks
    _simple("simple_gated_cfg2", (2, 32, 32, 1), 401,
            dict(kernel_size=5, rope_mode="spatiotemporal", gate_type="factored",
                 short_conv_size=4, short_conv_spatial_size=3),
            cssm_type="gated", embed_dim=8, kernel_size=5, gate_type="factored", seq_len=3,
            stem_layers=1, pool_type="max", pos_embed="spatiotemporal", num_classes=2),
    _simple("simple_gated_cfg1_two_stem_layers", (2, 32, 32, 1), 402,
            dict(kernel_size=1, rope_mode="spatiotemporal", gate_type="dense"),
            cssm_type="gated", embed_dim=8, kernel_size=1, gate_type="dense", seq_len=1,
            stem_layers=2, pool_type="mean", pos_embed="spatiotemporal", num_classes=2),
    _simple("simple_gdn_cfg3", (2, 32, 32, 1), 403,
            dict(kernel_size=5, rope_mode="mrope", gate_type="factored", qkv_conv_size=5,
                 delta_key_dim=4),
            cssm_type="gdn", embed_dim=8, kernel_size=5, gate_type="factored", seq_len=3,
            stem_layers=1, pool_type="max", pos_embed="mrope", qkv_conv_size=5, delta_key_dim=4,
            num_classes=2),
    _simple("simple_gdn_cfg4_clip", (2, 4, 16, 16, 3), 404,
            dict(kernel_size=5, rope_mode="spatiotemporal", gate_type="factored",
                 delta_key_dim=4),
            cssm_type="gdn", embed_dim=8, kernel_size=5, gate_type="factored",
            stem_mode="pathtracker", pool_type="mean", pos_embed="spatiotemporal",
            delta_key_dim=4, num_classes=2),
    # ---- CSSM-SHViT around the gated mixer (BASELINE configs[4]: T = 1, kernel_size 1)
    _shvit_block("shvit_block_stage2_14", (2, 14, 14, 32), 501, num_timesteps=1, kernel_size=1,
                 short_conv_spatial_size=0, gate_type="factored"),
    _shvit_block("shvit_block_stage3_7_T3_ks3", (2, 7, 7, 32), 502, num_timesteps=3, kernel_size=3,
                 gate_type="factored", rope_mode="spatiotemporal"),
    _shvit_block("shvit_block_no_posconv_no_dwconv", (2, 8, 8, 32), 503, num_timesteps=2,
                 kernel_size=3, gate_type="dense", use_pos_conv=False, use_dwconv=False),
    _shvit("shvit_tiny_64", (2, 64, 64, 3), 511, embed_dims=(32, 32, 64, 64), depths=(1, 2, 2, 1),
           num_classes=10, num_timesteps=1, kernel_sizes=(1, 1, 1, 1), short_conv_spatial_size=0),
    _shvit("shvit_tiny_T2_ks3_meanpool", (2, 32, 32, 3), 512, embed_dims=(32, 32, 32, 64),
           depths=(1, 1, 1, 1), num_classes=5, num_timesteps=2, kernel_sizes=(3, 3, 3, 3),
           head_pool="mean"),
    _shvit("shvit_s1_224_cfg5", (2, 224, 224, 3), 513, seeded=5130,
           num_timesteps=1, kernel_sizes=(1, 1, 1, 1), short_conv_spatial_size=0, **_S1),
]

BY_NAME = {c["name"]: c for c in CASES}
