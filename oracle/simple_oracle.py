"""CPU restatement (NumPy) of the SimpleCSSM model forward: stem -> CSSM block + residual ->
last-frame readout -> logits.

TEST INFRASTRUCTURE ONLY (same rule as cssm_oracle.py: only tests, the smoke check and the CPU
legs of the benchmark may import it).  PINNED like the block oracle: tests/test_reference_pin.py
compares it with outputs of the reference's own, unmodified src/models/simple_cssm.py run on
NumPy stand-ins for jax / flax.linen (tests/golden/ref/simple_*.npz), to 1e-9.

Reference lines followed (paths inside drewlinsley/CSSM):
  src/models/simple_cssm.py:86-157   fields and defaults
  src/models/simple_cssm.py:238-241  a 4-D image batch is repeated over seq_len frames
  src/models/simple_cssm.py:244-277  stem ('default': [conv3x3 SAME -> act -> norm -> 2x2 max-pool]
                                     per layer with stem_norm_order='post'; 'pathtracker': conv1x1
                                     -> act -> norm, no pooling)
  src/models/simple_cssm.py:318-482  block construction and  x = x + cssm(x)
  src/models/simple_cssm.py:523-556  frame_readout='last', readout_norm 'pre'/'post', spatial
                                     pool (mean / max), norm_post, Dense head
Flax conventions honoured: Conv is cross-correlation with HWIO kernels and 'SAME' zero padding
((k-1)//2 low, k//2 high); LayerNorm normalises the last axis with eps 1e-6 and the variance
computed as E[x^2] - E[x]^2, then scale and bias; nn.softplus is logaddexp(x, 0); max_pool
with 'SAME' padding pads with -inf on the high side when a dimension is odd.
"""
from __future__ import annotations

import inspect

import numpy as np

from . import cssm_oracle as orc


def layer_norm(x, p, eps=1e-6):
    x = np.asarray(x, np.float64)
    mu = x.mean(-1, keepdims=True)
    var = np.maximum((x * x).mean(-1, keepdims=True) - mu * mu, 0.0)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(p["scale"], np.float64) + np.asarray(p["bias"], np.float64)


def conv2d_same(x, p):
    """x (N,H,W,Cin), kernel (k,k,Cin,Cout): cross-correlation, zero 'SAME' padding."""
    x = np.asarray(x, np.float64)
    w = np.asarray(p["kernel"], np.float64)
    k = w.shape[0]
    lo, hi = (k - 1) // 2, k // 2
    N, H, W, _ = x.shape
    xp = np.pad(x, ((0, 0), (lo, hi), (lo, hi), (0, 0)))
    y = np.zeros((N, H, W, w.shape[-1]))
    for i in range(k):
        for j in range(k):
            y += xp[:, i:i + H, j:j + W, :] @ w[i, j]
    return y + np.asarray(p["bias"], np.float64)


def max_pool_2x2_same(x):
    N, H, W, C = x.shape
    ph, pw = H % 2, W % 2
    if ph or pw:
        x = np.pad(x, ((0, 0), (0, ph), (0, pw), (0, 0)), constant_values=-np.inf)
    N, H, W, C = x.shape
    return x.reshape(N, H // 2, 2, W // 2, 2, C).max(axis=(2, 4))


def stem_forward(params, frames, *, stem_mode="default", stem_layers=2):
    """frames (N,H,W,Cin) -> (N,H',W',embed_dim), stem_norm_order='post', act softplus,
    norm 'layer'."""
    x = np.asarray(frames, np.float64)
    if stem_mode == "pathtracker":
        x = conv2d_same(x, params["conv1"])
        return layer_norm(orc.softplus(x), params["norm1"])
    for i in range(stem_layers):
        x = conv2d_same(x, params[f"conv{i + 1}"])
        x = layer_norm(orc.softplus(x), params[f"norm{i + 1}"])
        x = max_pool_2x2_same(x)
    return x


def readout_forward(params, x_last, *, pool_type="mean", readout_norm="pre"):
    """x_last (B,H,W,C) -> logits (B,num_classes)."""
    x = np.asarray(x_last, np.float64)
    if readout_norm == "pre":
        x = orc.softplus(layer_norm(x, params["norm_pre"]))
    else:
        x = layer_norm(orc.softplus(x), params["norm_pre"])
    x = x.max(axis=(1, 2)) if pool_type == "max" else x.mean(axis=(1, 2))
    x = layer_norm(x, params["norm_post"])
    return x @ np.asarray(params["head"]["kernel"], np.float64) + np.asarray(params["head"]["bias"], np.float64)


def simple_forward(params, x, *, cssm_type="gated", seq_len=8, stem_mode="default", stem_layers=2,
                   pool_type="mean", readout_norm="pre", block_kwargs=None,
                   return_intermediates=False):
    """SimpleCSSM inference forward with depth 1, frame_readout 'last', act softplus, norm 'layer'.
    x: (B,H,W,Cin) images (repeated over seq_len) or (B,T,H,W,Cin) clips.  block_kwargs go to
    cssm_oracle.gated_forward / gdn_forward (kernel_size, rope_mode, gate_type, ...)."""
    x = np.asarray(x, np.float64)
    if x.ndim == 4:
        x = np.repeat(x[:, None], seq_len, axis=1)
    B, T = x.shape[:2]
    f = stem_forward(params, x.reshape((B * T,) + x.shape[2:]), stem_mode=stem_mode,
                     stem_layers=stem_layers)
    f = f.reshape((B, T) + f.shape[1:])
    kw = dict(block_kwargs or {})
    if cssm_type == "gated":
        y = orc.gated_forward(params["cssm_0"], f, **kw)
    elif cssm_type == "gdn":
        y = orc.gdn_forward(params["cssm_0"], f, **kw)
    elif cssm_type in _SCALAR_BLOCKS:
        fwd = _SCALAR_BLOCKS[cssm_type][0]
        accepted = set(inspect.signature(fwd).parameters)
        y = fwd(params["cssm_0"], f, **{k: v for k, v in kw.items() if k in accepted})
    else:
        raise ValueError(cssm_type)
    post = f + y
    logits = readout_forward(params, post[:, -1], pool_type=pool_type, readout_norm=readout_norm)
    if return_intermediates:
        return logits, {"stem": f, "post_cssm_last": post[:, -1]}
    return logits


def _init_nogate(seed, C, H, W, *, kernel_size=11, bias_scale=0.0):
    rng = np.random.default_rng(seed)
    return {"kernel": (0.3 * rng.standard_normal((C, kernel_size, kernel_size))).astype(np.float32),
            "out_proj": {"kernel": (rng.standard_normal((C, C)) / np.sqrt(C)).astype(np.float32),
                         "bias": (bias_scale * rng.standard_normal(C)).astype(np.float32)}}


# CSSM_REGISTRY names (simple_cssm.py:21-60) of the scalar-scan blocks -> (forward, init)
_SCALAR_BLOCKS = {"no_gate": (orc.nogate_forward, _init_nogate),
                  "add_kqv_1": (orc.additive1_forward, orc.init_additive1_params),
                  "deltanet": (orc.deltanet_forward, orc.init_deltanet_params)}


def init_simple_params(seed, *, cin, embed_dim, H, W, num_classes=2, cssm_type="gated",
                       stem_mode="default", stem_layers=2, bias_scale=0.1, block_kwargs=None):
    """Seeded stand-ins for the Flax initialisers (lecun-normal conv / dense kernels; LayerNorm
    scale 1 and bias 0, both perturbed when bias_scale > 0 so that indexing bugs show).
    H, W: size of the BLOCK input (after the stem)."""
    rng = np.random.default_rng(seed)
    p = {}

    def norm(c):
        return {"scale": (1.0 + bias_scale * rng.standard_normal(c)).astype(np.float32),
                "bias": (bias_scale * rng.standard_normal(c)).astype(np.float32)}

    def conv(k, ci, co):
        return {"kernel": (rng.standard_normal((k, k, ci, co)) / np.sqrt(k * k * ci)).astype(np.float32),
                "bias": (bias_scale * rng.standard_normal(co)).astype(np.float32)}

    if stem_mode == "pathtracker":
        p["conv1"], p["norm1"] = conv(1, cin, embed_dim), norm(embed_dim)
    else:
        ci = cin
        for i in range(stem_layers):
            p[f"conv{i + 1}"], p[f"norm{i + 1}"] = conv(3, ci, embed_dim), norm(embed_dim)
            ci = embed_dim
    if cssm_type in _SCALAR_BLOCKS:
        init = _SCALAR_BLOCKS[cssm_type][1]
    else:
        init = orc.init_gated_params if cssm_type == "gated" else orc.init_gdn_params
    accepted = set(inspect.signature(init).parameters)
    kw = {k: v for k, v in (block_kwargs or {}).items() if k in accepted}
    p["cssm_0"] = init(seed + 1, embed_dim, H, W, bias_scale=bias_scale, **kw)
    p["norm_pre"], p["norm_post"] = norm(embed_dim), norm(embed_dim)
    p["head"] = {"kernel": (rng.standard_normal((embed_dim, num_classes)) / np.sqrt(embed_dim)).astype(np.float32),
                 "bias": (bias_scale * rng.standard_normal(num_classes)).astype(np.float32)}
    return p
