"""Multi-threaded CPU restatement (PyTorch-CPU, float32) of the gated block forward.

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
