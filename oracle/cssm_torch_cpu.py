"""Multi-threaded CPU restatement (PyTorch-CPU, float32) of the gated and GDN block forwards
and of the SimpleCSSM model around them.

TEST / BASELINE INFRASTRUCTURE ONLY: this is the timed stand-in for "the reference on the
host cores" (the reference itself needs JAX, which is not installable here).  It follows
the same reference lines as oracle/cssm_oracle.py (src/models/cssm.py:476-585) op for op
— Dense, depthwise convs, SiLU, rfft2, gates, recurrence, irfft2, SiLU gate, Dense — using
torch's threaded CPU kernels, and is checked against the NumPy oracle in tests/.
PARITY UNPINNED against the JAX reference for the same reason as the NumPy oracle.
The recurrence is the direct complex form h_t = A_t h_{t-1} + U_t (the reference runs the
same recurrence as a log-space associative scan, which costs it more passes)."""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from . import cssm_oracle as orc


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def gated_forward_torch(params, x, *, kernel_size, rope_mode="none", rope_base=10000.0,
                        spectral_rho=0.999, short_conv_size=4, short_conv_spatial_size=3,
                        gate_type="dense"):
    """x: (B,T,H,W,C) float32 torch CPU tensor -> (B,T,H,W,C)."""
    B, T, H, W, C = x.shape
    Wf = W // 2 + 1
    if rope_mode != "none":
        ft, fh, fw = orc.rope_axis_freqs(C, rope_mode, rope_base)
        th = (np.arange(T)[:, None, None, None] * ft + np.arange(H)[None, :, None, None] * fh
              + np.arange(W)[None, None, :, None] * fw)
        c, s = _t(np.cos(th).astype(np.float32)), _t(np.sin(th).astype(np.float32))
        xe, xo = x[..., 0::2], x[..., 1::2]
        x = torch.stack([xe * c - xo * s, xe * s + xo * c], dim=-1).reshape(B, T, H, W, C)
    p = params
    xz = x.reshape(-1, C) @ _t(p["in_proj"]["kernel"]) + _t(p["in_proj"]["bias"])
    xz = xz.reshape(B, T, H, W, 2 * C)
    xm, z = xz[..., :C], xz[..., C:]
    if short_conv_spatial_size > 0:
        k = short_conv_spatial_size
        w = _t(p["short_conv_spatial"]["kernel"]).permute(3, 2, 0, 1).contiguous()   # (C,1,k,k)
        xm = F.conv2d(xm.reshape(B * T, H, W, C).permute(0, 3, 1, 2), w,
                      _t(p["short_conv_spatial"]["bias"]), padding=(k - 1) // 2, groups=C)
        xm = xm.permute(0, 2, 3, 1).reshape(B, T, H, W, C)
    if short_conv_size > 0:
        k = short_conv_size
        w = _t(p["short_conv_temporal"]["kernel"])        # (k,1,C)
        xp = F.pad(xm, (0, 0, 0, 0, 0, 0, k - 1, 0))
        acc = _t(p["short_conv_temporal"]["bias"]).expand_as(xm).clone()
        for j in range(k):
            acc = acc + xp[:, j:j + T] * w[j, 0]
        xm = acc
    xm = F.silu(xm)
    K = _t(orc.goom_floor(orc.spectral_kernel(p["kernel"], H, W, spectral_rho)).astype(np.complex64))
    U = torch.fft.rfft2(xm.permute(0, 1, 4, 2, 3), dim=(3, 4))      # (B,T,C,H,Wf)
    ctx = xm.mean(dim=(2, 3))

    def gate(name):
        if gate_type == "factored":
            gh = ctx @ _t(p[f"{name}_h"]["kernel"]) + _t(p[f"{name}_h"]["bias"])
            gw = ctx @ _t(p[f"{name}_w"]["kernel"]) + _t(p[f"{name}_w"]["bias"])
            return (gh[..., :, None] * gw[..., None, :]).reshape(B, T, 1, H, Wf)
        return (ctx @ _t(p[name]["kernel"]) + _t(p[name]["bias"])).reshape(B, T, 1, H, Wf)

    delta = F.softplus(gate("delta_proj"))
    Bg, Cg = gate("B_proj"), gate("C_proj")
    BU = U * Bg
    small = BU.abs() < 1e-7
    BU = torch.where(small, torch.full_like(BU, 1e-7), BU)
    Uin = (delta + 1e-8) * BU
    decay = torch.exp(-delta)
    h = torch.zeros_like(Uin[:, 0])
    outs = []
    for t in range(T):
        h = (K[None] * decay[:, t]) * h + Uin[:, t]
        outs.append(h * Cg[:, t])
    Y = torch.stack(outs, dim=1)
    ssm = torch.fft.irfft2(Y, s=(H, W), dim=(3, 4)).permute(0, 1, 3, 4, 2)
    out = (ssm * F.silu(z)).reshape(-1, C) @ _t(p["out_proj"]["kernel"]) + _t(p["out_proj"]["bias"])
    return out.reshape(B, T, H, W, C)


def _rope_torch(x, rope_mode, rope_base):
    B, T, H, W, C = x.shape
    if rope_mode == "none":
        return x
    ft, fh, fw = orc.rope_axis_freqs(C, rope_mode, rope_base)
    th = (np.arange(T)[:, None, None, None] * ft + np.arange(H)[None, :, None, None] * fh
          + np.arange(W)[None, None, :, None] * fw)
    c, s = _t(np.cos(th).astype(np.float32)), _t(np.sin(th).astype(np.float32))
    xe, xo = x[..., 0::2], x[..., 1::2]
    return torch.stack([xe * c - xo * s, xe * s + xo * c], dim=-1).reshape(B, T, H, W, C)


def _dense_t(x, p):
    return x @ _t(p["kernel"]) + _t(p["bias"])


def _tconv_silu(x, p, k):
    """Causal depthwise temporal conv (left pad k-1) then SiLU; x (B,T,H,W,C)."""
    T = x.shape[1]
    w = _t(p["kernel"])
    xp = F.pad(x, (0, 0, 0, 0, 0, 0, k - 1, 0))
    acc = _t(p["bias"]).expand_as(x).clone()
    for j in range(k):
        acc = acc + xp[:, j:j + T] * w[j, 0]
    return F.silu(acc)


def gdn_forward_torch(params, x, *, delta_key_dim=4, kernel_size=11, rope_mode="none",
                      rope_base=10000.0, spectral_rho=0.999, gate_type="factored",
                      short_conv_size=4, output_norm="rms", use_input_gates=True,
                      output_gate_act="silu", use_spectral_l2_norm=True, qkv_conv_size=1,
                      no_spectral_clamp=False):
    """GatedDeltaNetCSSM general path (src/models/cssm.py:4685-5141) in float32 / complex64 on the
    host cores.  Like the reference it materialises M_t and Delta_t per bin; the scan is the
    direct recurrence S_t = M_t S_{t-1} + Delta_t with the 1e-7 magnitude floor on M and Delta."""
    B, T, H, W, C = x.shape
    Wf, dk = W // 2 + 1, delta_key_dim
    nh = C // dk
    p = params
    x = _rope_torch(x, rope_mode, rope_base)
    W_hat = _t(orc.spectral_kernel(p["kernel"], H, W, spectral_rho,
                                   squash=not no_spectral_clamp).astype(np.complex64))
    xf = x.reshape(B * T, H, W, C)
    qin = xf
    if qkv_conv_size > 1:
        k = qkv_conv_size
        w = _t(p["qkv_dw"]["kernel"]).permute(3, 2, 0, 1).contiguous()
        qin = F.conv2d(xf.permute(0, 3, 1, 2), w, _t(p["qkv_dw"]["bias"]), padding=(k - 1) // 2,
                       groups=C).permute(0, 2, 3, 1)
    qkv = _dense_t(qin.reshape(-1, C), p["qkv_proj"]).reshape(B, T, H, W, 3 * C)
    q_in, k_in, v_in = qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:]
    if short_conv_size > 0:
        q_in = _tconv_silu(q_in, p["short_conv_q"], short_conv_size)
        k_in = _tconv_silu(k_in, p["short_conv_k"], short_conv_size)
        v_in = _tconv_silu(v_in, p["short_conv_v"], short_conv_size)
    ctx = x.mean(dim=(2, 3)) + _t(orc.temporal_ctx_code(T, C, rope_base).astype(np.float32))[None]

    def gate(name, bounded=False, spatial=False):
        Wd = W if spatial else Wf
        if gate_type == "factored":
            raw = torch.sigmoid(_dense_t(ctx, p[f"{name}_h"])[..., :, None]
                                + _dense_t(ctx, p[f"{name}_w"])[..., None, :])
        else:
            raw = torch.sigmoid(_dense_t(ctx, p[name])).reshape(B, T, H, Wd)
        if spatial:
            return raw.reshape(B, T, H, W, 1)
        raw = raw.reshape(B, T, 1, H, Wf)
        return 0.1 + 0.89 * raw if bounded else raw

    if use_input_gates:
        k_in = k_in * gate("B_k", spatial=True)
        v_in = v_in * gate("B_v", spatial=True)
    gate_val = _dense_t(xf.reshape(-1, C), p["gate_proj"]).reshape(B, T, H, W, C)
    gate_val = F.silu(gate_val) if output_gate_act == "silu" else torch.sigmoid(gate_val)
    alpha, beta = gate("alpha", bounded=True), gate("beta")

    def spec(a):
        a = a.reshape(B, T, H, W, nh, dk).permute(0, 1, 4, 5, 2, 3)
        return torch.fft.rfft2(a, dim=(4, 5))                                   # (B,T,nh,dk,H,Wf)

    q_s, k_s, v_s = spec(q_in), spec(k_in), spec(v_in)

    def l2(z):
        if not use_spectral_l2_norm:
            return z
        return z / torch.sqrt((z.abs() ** 2).sum(dim=(4, 5), keepdim=True) + 1e-6)

    k_s = l2(k_s)
    k_n = k_s / torch.sqrt((k_s.abs() ** 2).sum(dim=3, keepdim=True) + 1e-6)
    q_n = l2(q_s)
    a_bc, b_bc = alpha[:, :, :, None, None], beta[:, :, :, None, None]
    k_outer = k_n[:, :, :, :, None] * torch.conj(k_n[:, :, :, None, :])
    eye = torch.eye(dk).reshape(1, 1, 1, dk, dk, 1, 1)
    M = a_bc * W_hat[None, None, :, None, None] * (eye - b_bc * k_outer)
    Delta = b_bc * (v_s[:, :, :, :, None] * torch.conj(k_n[:, :, :, None, :]))

    def floor(z):
        return torch.where(z.abs() < 1e-7, torch.full_like(z, 1e-7), z)

    M, Delta = floor(M), floor(Delta)
    s = torch.zeros((B, nh, dk, dk, H, Wf), dtype=torch.complex64)
    outs = []
    for t in range(T):
        s = torch.einsum("bhijyx,bhvjyx->bhviyx", M[:, t], s) + Delta[:, t]
        outs.append((s * q_n[:, t, :, None]).sum(dim=3))                        # (B,nh,v,H,Wf)
    o_hat = torch.stack(outs, dim=1).reshape(B, T, C, H, Wf)
    o = torch.fft.irfft2(o_hat, s=(H, W), dim=(3, 4)).permute(0, 1, 3, 4, 2)
    if output_norm == "rms":
        o = o * torch.rsqrt((o * o).mean(dim=-1, keepdim=True) + 1e-6) * _t(p["rms_scale"])
    out = _dense_t((o * gate_val).reshape(-1, C), p["output_proj"])
    return out.reshape(B, T, H, W, C)


def _layer_norm_t(x, p):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x * x).mean(dim=-1, keepdim=True) - mu * mu).clamp_min(0.0)
    return (x - mu) * torch.rsqrt(var + 1e-6) * _t(p["scale"]) + _t(p["bias"])


def simple_forward_torch(params, x, *, cssm_type="gated", seq_len=8, stem_mode="default",
                         stem_layers=2, pool_type="mean", readout_norm="pre", block_kwargs=None):
    """SimpleCSSM inference forward (src/models/simple_cssm.py:173-558) on the host cores, op for
    op as the reference runs it: an image batch is first repeated over seq_len frames and the
    stem then runs on all B*T frames; the block produces all T frames; the readout takes the
    last.  x: (B,H,W,Cin) or (B,T,H,W,Cin) float32 torch CPU tensor -> logits (B,num_classes)."""
    p = params
    if x.dim() == 4:
        x = x[:, None].expand(-1, seq_len, -1, -1, -1)
    B, T = x.shape[:2]
    f = x.reshape((B * T,) + tuple(x.shape[2:])).permute(0, 3, 1, 2)
    if stem_mode == "pathtracker":
        w = _t(p["conv1"]["kernel"]).permute(3, 2, 0, 1).contiguous()
        f = F.conv2d(f, w, _t(p["conv1"]["bias"])).permute(0, 2, 3, 1)
        f = _layer_norm_t(F.softplus(f), p["norm1"])
    else:
        for i in range(stem_layers):
            w = _t(p[f"conv{i + 1}"]["kernel"]).permute(3, 2, 0, 1).contiguous()
            f = F.conv2d(f, w, _t(p[f"conv{i + 1}"]["bias"]), padding=1).permute(0, 2, 3, 1)
            f = _layer_norm_t(F.softplus(f), p[f"norm{i + 1}"]).permute(0, 3, 1, 2)
            f = F.max_pool2d(f, 2, 2, ceil_mode=True)
        f = f.permute(0, 2, 3, 1)
    f = f.reshape((B, T) + tuple(f.shape[1:])).contiguous()
    kw = dict(block_kwargs or {})
    y = (gated_forward_torch if cssm_type == "gated" else gdn_forward_torch)(p["cssm_0"], f, **kw)
    z = (f + y)[:, -1]
    if readout_norm == "pre":
        z = F.softplus(_layer_norm_t(z, p["norm_pre"]))
    else:
        z = _layer_norm_t(F.softplus(z), p["norm_pre"])
    z = z.amax(dim=(1, 2)) if pool_type == "max" else z.mean(dim=(1, 2))
    z = _layer_norm_t(z, p["norm_post"])
    return z @ _t(p["head"]["kernel"]) + _t(p["head"]["bias"])


# ------------------------------------------------------------------ CSSM-SHViT (timed CPU leg)
def _conv_same(x, kernel, bias, stride=1, groups=1):
    """'SAME' conv as XLA pads it (total = (ceil(n/s)-1)*s + k - n, the smaller half first).
    x (N,C,H,W); kernel HWIO."""
    kh, kw = kernel.shape[:2]
    H, W = x.shape[-2:]
    th = max((-(-H // stride) - 1) * stride + kh - H, 0)
    tw = max((-(-W // stride) - 1) * stride + kw - W, 0)
    x = F.pad(x, (tw // 2, tw - tw // 2, th // 2, th - th // 2))
    return F.conv2d(x, _t(kernel).permute(3, 2, 0, 1).contiguous(), None if bias is None else _t(bias),
                    stride=stride, groups=groups)


def _convbn_t(x, p, s, stride):
    y = _conv_same(x, p["conv"]["kernel"], None, stride)
    return F.batch_norm(y, _t(s["bn"]["mean"]), _t(s["bn"]["var"]), _t(p["bn"]["scale"]), _t(p["bn"]["bias"]),
                        training=False, eps=1e-5)


def _ln_cl(x, p):
    return F.layer_norm(x, x.shape[-1:], _t(p["scale"]), _t(p["bias"]), eps=1e-6)


def _dw_cl(x, p):
    """Depthwise 'SAME' conv on a channels-last tensor."""
    return _conv_same(x.permute(0, 3, 1, 2), p["kernel"], p["bias"], groups=x.shape[-1]).permute(0, 2, 3, 1)


def _mlp_t(x, p, use_dwconv):
    h = F.gelu(F.linear(x, _t(p["fc1"]["kernel"]).T, _t(p["fc1"]["bias"])), approximate="tanh")
    if use_dwconv:
        h = h + _dw_cl(h, p["dwconv"]["dwconv"])
    return F.linear(h, _t(p["fc2"]["kernel"]).T, _t(p["fc2"]["bias"]))


def shvit_forward_torch(params, stats, x, *, embed_dims=(64, 128, 256, 384), depths=(1, 2, 2, 1),
                        use_cssm_stages=(False, False, True, True), num_timesteps=8,
                        kernel_sizes=(15, 15, 5, 3), use_pos_conv=True, use_dwconv=True,
                        head_pool="max", gate_type="factored", **gated_kw):
    """CSSMSHViT inference forward (src/models/cssm_shvit.py:324-460, gated mixers, image input) in
    float32 on the host cores, op for op as the reference runs it (the image is repeated over
    num_timesteps in front of every CSSM block and all T frames go through the mixer).
    x: (B,H,W,3) float32 torch CPU tensor -> logits (B,num_classes)."""
    p, s = params, stats
    y = x.permute(0, 3, 1, 2)
    y = F.gelu(_convbn_t(y, p["patch_embed"]["ConvBN_0"], s["patch_embed"]["ConvBN_0"], 2), approximate="tanh")
    y = _convbn_t(y, p["patch_embed"]["ConvBN_1"], s["patch_embed"]["ConvBN_1"], 2)
    for st in range(4):
        if st > 0:
            y = _convbn_t(y, p[f"downsample{st}"]["ConvBN_0"], s[f"downsample{st}"]["ConvBN_0"], 2)
        v = y.permute(0, 2, 3, 1)
        for b in range(depths[st]):
            bp = p[f"stage{st}_block{b}"]
            if use_cssm_stages[st]:
                B, H, W, C = v.shape
                T = num_timesteps
                xt = v[:, None].expand(-1, T, -1, -1, -1)
                h = F.layer_norm(xt, xt.shape[1:], eps=1e-6) * _t(bp["norm1"]["scale"]) + _t(bp["norm1"]["bias"])
                if use_pos_conv:
                    h = h + _dw_cl(h.reshape(B * T, H, W, C), bp["pos_conv"]).reshape(B, T, H, W, C)
                m = gated_forward_torch(bp["cssm"], h.contiguous(), kernel_size=kernel_sizes[st],
                                        gate_type=gate_type, **gated_kw)
                v = v + m[:, -1]
                v = v + _mlp_t(_ln_cl(v, bp["norm2"]), bp["mlp"], use_dwconv)
            else:
                h = F.gelu(_dw_cl(_ln_cl(v, bp["norm1"]), bp["dwconv"]["dwconv"]), approximate="tanh")
                v = v + F.linear(h, _t(bp["pwconv"]["kernel"]).T, _t(bp["pwconv"]["bias"]))
                v = v + _mlp_t(_ln_cl(v, bp["norm2"]), bp["mlp"], False)
        y = v.permute(0, 3, 1, 2)
    v = _ln_cl(y.permute(0, 2, 3, 1), p["norm"])
    pooled = v.amax(dim=(1, 2)) if head_pool == "max" else v.mean(dim=(1, 2))
    return pooled @ _t(p["head"]["kernel"]) + _t(p["head"]["bias"])
