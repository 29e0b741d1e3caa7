"""CPU restatement (NumPy, fp64) of the CSSM-SHViT inference forward around the gated mixer.

TEST INFRASTRUCTURE ONLY (the checker of the CUDA path; nothing in `cssm_b200/` imports it).
Pinned: tests/test_reference_pin.py compares it with outputs of the reference's own, unmodified
`src/models/cssm_shvit.py` / `shvit.py` (tests/golden/ref/shvit_*.npz).

Reference lines followed (paths inside drewlinsley/CSSM):
  src/models/shvit.py:34-61      ConvBN: Conv(k, stride, 'SAME', no bias) + BatchNorm (running stats)
  src/models/shvit.py:64-81      PatchEmbed: ConvBN(E/2, 3, s2) -> gelu -> ConvBN(E, 3, s2)
  src/models/shvit.py:84-95      Downsample: ConvBN(out, 3, s2)
  src/models/shvit.py:98-116     DWConv (depthwise 'SAME', bias)
  src/models/shvit.py:154-182    Mlp: fc1 -> gelu -> [x + DWConv3(x)] -> fc2
  src/models/shvit.py:219-262    ConvBlock: LN -> DWConv7 -> gelu -> Dense -> +res; LN -> Mlp -> +res
  src/models/cssm_shvit.py:19-266   CSSMSHViTBlock (image input, cssm_type 'gated')
  src/models/cssm_shvit.py:269-460  CSSMSHViT; :465-474 cssm_shvit_s1
Conventions: 'SAME' with stride s pads total = (ceil(n/s)-1)*s + k - n, the smaller half first
(for even n, k=3, s=2: nothing before, one after); jax.nn.gelu is the tanh form; BatchNorm
eps 1e-5, LayerNorm eps 1e-6; inference only (deterministic=True: DropPath is the identity).

`rnd` rounds where a model built with dtype=bfloat16 rounds (the output of every Conv / Dense /
norm / activation outside the mixer, which has no dtype field and computes in float32): the
identity gives the exact forward, `cssm_oracle.bf16_round` an emulation of the bf16 model.
"""
from __future__ import annotations

import numpy as np

from . import cssm_oracle as orc


def gelu_tanh(x):
    return 0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))


def same_pads(n, k, s):
    tot = max((-(-n // s) - 1) * s + k - n, 0)
    return tot // 2, tot - tot // 2


def conv2d(x, kernel, bias=None, stride=1):
    """Cross-correlation, HWIO kernel, 'SAME'.  x (N,H,W,Cin)."""
    kh, kw, ci, co = kernel.shape
    N, H, W, _ = x.shape
    ph, pw = same_pads(H, kh, stride), same_pads(W, kw, stride)
    xp = np.pad(x, ((0, 0), ph, pw, (0, 0)))
    Ho, Wo = -(-H // stride), -(-W // stride)
    y = np.zeros((N, Ho, Wo, co))
    for i in range(kh):
        for j in range(kw):
            y += xp[:, i:i + (Ho - 1) * stride + 1:stride, j:j + (Wo - 1) * stride + 1:stride] @ kernel[i, j]
    return y if bias is None else y + bias


def dwconv2d(x, p):
    """Depthwise 'SAME' conv, kernel (k,k,1,C) + bias."""
    k = p["kernel"].shape[0]
    N, H, W, C = x.shape
    lo, hi = same_pads(H, k, 1)
    xp = np.pad(x, ((0, 0), (lo, hi), same_pads(W, k, 1), (0, 0)))
    y = np.zeros_like(x)
    for i in range(k):
        for j in range(k):
            y += xp[:, i:i + H, j:j + W] * p["kernel"][i, j, 0]
    return y + p["bias"]


def conv_bn(x, p, s, stride, rnd):
    y = rnd(conv2d(x, p["conv"]["kernel"].astype(np.float64), None, stride))
    mean, var = s["bn"]["mean"].astype(np.float64), s["bn"]["var"].astype(np.float64)
    y = (y - mean) / np.sqrt(var + 1e-5) * p["bn"]["scale"] + p["bn"]["bias"]
    return rnd(y)


def layer_norm(x, p, axes=(-1,), eps=1e-6):
    mean = x.mean(axis=axes, keepdims=True)
    var = x.var(axis=axes, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * p["scale"] + p["bias"]


def mlp(x, p, use_dwconv, rnd):
    h = rnd(gelu_tanh(rnd(orc.dense(x, p["fc1"]))))
    if use_dwconv:
        h = rnd(h + rnd(dwconv2d(h, p["dwconv"]["dwconv"])))
    return rnd(orc.dense(h, p["fc2"]))


def conv_block(x, p, rnd):
    """shvit.py:219-262."""
    h = rnd(layer_norm(x, p["norm1"]))
    h = rnd(gelu_tanh(rnd(dwconv2d(h, p["dwconv"]["dwconv"]))))
    x = x + rnd(orc.dense(h, p["pwconv"]))
    h = rnd(layer_norm(x, p["norm2"]))
    return x + mlp(h, p["mlp"], False, rnd)


def cssm_block(x, p, *, num_timesteps, kernel_size, rnd=lambda a: a, use_pos_conv=True,
               use_dwconv=True, block_norm="global_layer", gate_type="factored",
               return_intermediates=False, **gated_kw):
    """CSSMSHViTBlock on an image batch x (B,H,W,C), cssm_type 'gated' (cssm_shvit.py:66-266):
    repeat over T, LayerNorm over (T,H,W,C) with per-channel scale / bias, x + dw3x3(x) per frame,
    GatedCSSM, last frame + residual, LayerNorm + Mlp + residual."""
    B, H, W, C = x.shape
    T = num_timesteps
    xt = np.repeat(x[:, None], T, axis=1)
    if block_norm == "global_layer":
        h = layer_norm(xt, p["norm1"], axes=(1, 2, 3, 4))
    elif block_norm == "temporal_layer":
        h = layer_norm(xt, p["norm1"], axes=(1, 4))
    else:
        h = layer_norm(xt, p["norm1"])
    h = rnd(h)
    if use_pos_conv:
        h = rnd(h + rnd(dwconv2d(h.reshape(B * T, H, W, C), p["pos_conv"])).reshape(h.shape))
    mixer_in = h
    y = orc.gated_forward(p["cssm"], h, kernel_size=kernel_size, gate_type=gate_type, **gated_kw)
    x1 = x + y[:, -1]
    h = rnd(layer_norm(x1, p["norm2"]))
    out = x1 + mlp(h, p["mlp"], use_dwconv, rnd)
    if return_intermediates:
        return out, dict(mixer_in=mixer_in, mixer_out=y, after_mixer=x1)
    return out


def shvit_forward(params, stats, x, *, embed_dims=(64, 128, 256, 384), depths=(1, 2, 2, 1),
                  use_cssm_stages=(False, False, True, True), num_timesteps=8,
                  kernel_sizes=(15, 15, 5, 3), rnd=lambda a: a, use_pos_conv=True, use_dwconv=True,
                  block_norm="global_layer", head_pool="max", return_intermediates=False,
                  **gated_kw):
    """CSSMSHViT.__call__(x, training=False) on images x (B,H,W,3) with cssm_type 'gated'
    (cssm_shvit.py:324-460).  gated_kw: rope_mode, gate_type, short_conv_size,
    short_conv_spatial_size, gate_activation_kind, spectral_rho of the mixers."""
    x = rnd(np.asarray(x, np.float64))
    pe, se = params["patch_embed"], stats["patch_embed"]
    x = conv_bn(x, pe["ConvBN_0"], se["ConvBN_0"], 2, rnd)
    x = rnd(gelu_tanh(x))
    x = conv_bn(x, pe["ConvBN_1"], se["ConvBN_1"], 2, rnd)
    inter = {"patch_embed": x}
    for s in range(4):
        if s > 0:
            x = conv_bn(x, params[f"downsample{s}"]["ConvBN_0"], stats[f"downsample{s}"]["ConvBN_0"], 2, rnd)
        for b in range(depths[s]):
            p = params[f"stage{s}_block{b}"]
            if use_cssm_stages[s]:
                x = cssm_block(x, p, num_timesteps=num_timesteps, kernel_size=kernel_sizes[s],
                               rnd=rnd, use_pos_conv=use_pos_conv, use_dwconv=use_dwconv,
                               block_norm=block_norm, **gated_kw)
            else:
                x = conv_block(x, p, rnd)
            inter[f"stage{s}_block{b}"] = x
    x = rnd(layer_norm(x, params["norm"]))
    pooled = x.max(axis=(1, 2)) if head_pool == "max" else x.mean(axis=(1, 2))
    logits = orc.dense(pooled, params["head"])
    if return_intermediates:
        inter["pooled"] = pooled
        return logits, inter
    return logits


# ------------------------------------------------------------- seeded weight trees
def init_shvit_params(seed, in_hw, *, embed_dims=(64, 128, 256, 384), depths=(1, 2, 2, 1),
                      use_cssm_stages=(False, False, True, True), kernel_sizes=(15, 15, 5, 3),
                      num_classes=1000, mlp_ratio=4.0, gate_type="factored", short_conv_size=4,
                      short_conv_spatial_size=3, use_pos_conv=True, use_dwconv=True, cin=3,
                      bias_scale=0.1):
    """-> (params, batch_stats), float32, names and shapes of the reference's tree
    (checked against the reference's own init in tests/test_reference_pin.py)."""
    rng = np.random.default_rng(seed)
    f32 = np.float32

    def vec(c, centre=0.0, scale=bias_scale):
        return (centre + scale * rng.standard_normal(c)).astype(f32)

    def norm(c):
        return {"scale": vec(c, 1.0), "bias": vec(c)}

    def dense(ci, co):
        return {"kernel": (rng.standard_normal((ci, co)) / np.sqrt(ci)).astype(f32), "bias": vec(co)}

    def dw(k, c):
        return {"kernel": (rng.standard_normal((k, k, 1, c)) / k).astype(f32), "bias": vec(c)}

    def convbn(ci, co):
        p = {"conv": {"kernel": (rng.standard_normal((3, 3, ci, co)) / np.sqrt(9 * ci)).astype(f32)},
             "bn": norm(co)}
        s = {"bn": {"mean": vec(co, 0.0, 0.2), "var": np.exp(vec(co, 0.0, 0.3)).astype(f32)}}
        return p, s

    params, stats = {}, {}
    E = embed_dims
    pe0, se0 = convbn(cin, E[0] // 2)
    pe1, se1 = convbn(E[0] // 2, E[0])
    params["patch_embed"] = {"ConvBN_0": pe0, "ConvBN_1": pe1}
    stats["patch_embed"] = {"ConvBN_0": se0, "ConvBN_1": se1}
    H, W = (-(-in_hw[0] // 4)), (-(-in_hw[1] // 4))
    for s in range(4):
        if s > 0:
            p, st = convbn(E[s - 1], E[s])
            params[f"downsample{s}"], stats[f"downsample{s}"] = {"ConvBN_0": p}, {"ConvBN_0": st}
            H, W = -(-H // 2), -(-W // 2)
        hid = int(E[s] * mlp_ratio)
        for b in range(depths[s]):
            if use_cssm_stages[s]:
                blk = {"norm1": norm(E[s]), "norm2": norm(E[s]),
                       "cssm": orc.init_gated_params(int(rng.integers(1 << 30)), E[s], H, W,
                                                     kernel_size=kernel_sizes[s], gate_type=gate_type,
                                                     short_conv_size=short_conv_size,
                                                     short_conv_spatial_size=short_conv_spatial_size,
                                                     bias_scale=bias_scale),
                       "mlp": {"fc1": dense(E[s], hid), "fc2": dense(hid, E[s])}}
                if use_pos_conv:
                    blk["pos_conv"] = dw(3, E[s])
                if use_dwconv:
                    blk["mlp"]["dwconv"] = {"dwconv": dw(3, hid)}
            else:
                blk = {"norm1": norm(E[s]), "dwconv": {"dwconv": dw(7, E[s])},
                       "pwconv": dense(E[s], E[s]), "norm2": norm(E[s]),
                       "mlp": {"fc1": dense(E[s], hid), "fc2": dense(hid, E[s])}}
            params[f"stage{s}_block{b}"] = blk
    params["norm"] = norm(E[3])
    params["head"] = dense(E[3], num_classes)
    return params, stats
