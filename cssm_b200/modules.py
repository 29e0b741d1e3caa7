"""Host-side mirrors of the reference's Flax modules for the two spectral token mixers.

`GatedCSSM` and `GatedDeltaNetCSSM` keep the reference's dataclass fields, defaults and
call signature (src/models/cssm.py:416-430, 443-454 and :4298-4338, 4340-4352) and its
parameter tree (Flax names, Dense kernels (in, out), conv kernels HWIO), so the same
`module.apply({'params': tree}, x)` call works.  The arithmetic runs in libcssm_b200.so
through the C ABI; torch is used only for device memory and streams.  Field combinations
the CUDA path has no kernel for raise NotImplementedError — nothing falls back to
PyTorch or the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import numpy as np
import torch

from . import _lib
from ._lib import (GATE_ACTS, GATE_TYPES, ROPE_MODES, GatedDesc, GatedWeights, GatedWsLayout,
                   GdnDesc, GdnWeights, check)


def _dev_f32(a, device) -> torch.Tensor:
    if isinstance(a, torch.Tensor):
        return a.detach().to(device=device, dtype=torch.float32).contiguous()
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a, dtype=np.float32))).to(device)


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(x):
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("x must be a CUDA torch.Tensor (use forward_host for host arrays); "
                        "cssm_b200 has no CPU path")
    if x.dtype != torch.float32:
        raise TypeError(f"x must be float32, got {x.dtype}")


class _Buffers:
    """Caches device byte buffers by (tag, size) so repeated calls do not reallocate."""

    def __init__(self, device):
        self.device = device
        self._b: Dict[str, torch.Tensor] = {}

    def get(self, tag: str, nbytes: int) -> torch.Tensor:
        t = self._b.get(tag)
        if t is None or t.numel() < nbytes:
            t = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=self.device)
            self._b[tag] = t
        return t


# ============================================================================ gated
@dataclass
class GatedCSSM:
    """Spectral Mamba block (reference: GatedCSSM, src/models/cssm.py:384-585)."""
    channels: int
    dense_mixing: bool = False
    block_size: int = 32
    mixing_rank: int = 0
    kernel_size: int = 15
    spectral_rho: float = 0.999
    gate_activation: str = "softplus"
    rope_mode: str = "none"
    gate_rank: int = 0
    rope_base: float = 10000.0
    concat_xy: bool = True
    position_independent_gates: bool = False
    short_conv_size: int = 4
    short_conv_spatial_size: int = 3
    gate_type: str = "dense"
    name: Optional[str] = None
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    # -- parameter tree -----------------------------------------------------------
    def param_shapes(self, H: int, W: int) -> Dict[str, Any]:
        """Names and shapes of the Flax parameter tree for an (H, W) input."""
        Cc, Wf = self.channels, W // 2 + 1
        s: Dict[str, Any] = {
            "in_proj": {"kernel": (Cc, 2 * Cc), "bias": (2 * Cc,)},
            "kernel": (Cc, self.kernel_size, self.kernel_size),
            "out_proj": {"kernel": (Cc, Cc), "bias": (Cc,)},
        }
        if self.short_conv_spatial_size > 0:
            k = self.short_conv_spatial_size
            s["short_conv_spatial"] = {"kernel": (k, k, 1, Cc), "bias": (Cc,)}
        if self.short_conv_size > 0:
            s["short_conv_temporal"] = {"kernel": (self.short_conv_size, 1, Cc), "bias": (Cc,)}
        for n in ("delta_proj", "B_proj", "C_proj"):
            if self.gate_type == "factored":
                s[f"{n}_h"] = {"kernel": (Cc, H), "bias": (H,)}
                s[f"{n}_w"] = {"kernel": (Cc, Wf), "bias": (Wf,)}
            else:
                s[n] = {"kernel": (Cc, H * Wf), "bias": (H * Wf,)}
        return s

    def init(self, seed: int, x_shape, bias_scale: float = 0.0) -> Dict[str, Any]:
        """Random-init variables {'params': tree} (NumPy-seeded stand-ins for the Flax
        initialisers: lecun-normal Dense/Conv kernels, N(0, 0.02) spectral kernel)."""
        _, _, H, W, Cc = x_shape
        assert Cc == self.channels
        rng = np.random.default_rng(seed)

        def make(shape_tree):
            out = {}
            for k, v in shape_tree.items():
                if isinstance(v, dict):
                    kern = v["kernel"]
                    fan_in = int(np.prod(kern[:-1])) if len(kern) != 4 else kern[0] * kern[1]
                    if len(kern) == 3:      # temporal depthwise (k, 1, C)
                        fan_in = kern[0]
                    out[k] = {"kernel": (rng.standard_normal(kern) / np.sqrt(fan_in)).astype(np.float32),
                              "bias": (bias_scale * rng.standard_normal(v["bias"])).astype(np.float32)}
                else:
                    out[k] = (0.02 * rng.standard_normal(v)).astype(np.float32)
            return out

        return {"params": make(self.param_shapes(H, W))}

    # -- validation ---------------------------------------------------------------
    def _check_fields(self):
        if self.dense_mixing or self.mixing_rank > 0:
            raise NotImplementedError("GatedCSSM: only the depthwise path (dense_mixing=False) "
                                      "has a CUDA kernel")
        if self.gate_type not in GATE_TYPES:
            raise NotImplementedError(f"gate_type={self.gate_type!r}")
        if self.rope_mode not in ROPE_MODES:
            raise NotImplementedError(f"rope_mode={self.rope_mode!r}")

    def _desc(self, shape) -> GatedDesc:
        B, T, H, W, Cc = shape
        if Cc != self.channels:
            raise ValueError(f"x has {Cc} channels, module has {self.channels}")
        return GatedDesc(B, T, H, W, Cc, self.kernel_size, ROPE_MODES[self.rope_mode],
                         float(self.rope_base), float(self.spectral_rho),
                         GATE_ACTS.get(self.gate_activation, 0), self.short_conv_size,
                         self.short_conv_spatial_size, GATE_TYPES[self.gate_type])

    # -- binding of a parameter tree ---------------------------------------------
    def bind(self, variables, device="cuda") -> "BoundGated":
        self._check_fields()
        return BoundGated(self, variables["params"] if "params" in variables else variables,
                          torch.device(device))

    def apply(self, variables, x, injected_qkv_spatial=None):
        """Flax-style call: y = module.apply({'params': tree}, x).  x: (B,T,H,W,C) float32
        CUDA tensor.  `injected_qkv_spatial` is accepted and ignored, as in the reference."""
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            _require_cuda(x)
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


class BoundGated:
    """A GatedCSSM with its weights resident on one GPU and its plan/workspace cached."""

    def __init__(self, mod: GatedCSSM, params, device):
        self.mod = mod
        self.device = device
        self.variables_ref = None
        self.L = _lib.lib()
        p = params
        self.t: Dict[str, torch.Tensor] = {}

        def put(name, arr):
            self.t[name] = _dev_f32(arr, device)
            return self.t[name].data_ptr()

        w = GatedWeights()
        w.in_proj_kernel = put("ipk", p["in_proj"]["kernel"])
        w.in_proj_bias = put("ipb", p["in_proj"]["bias"])
        if mod.short_conv_spatial_size > 0:
            w.conv_sp_kernel = put("csk", p["short_conv_spatial"]["kernel"])
            w.conv_sp_bias = put("csb", p["short_conv_spatial"]["bias"])
        if mod.short_conv_size > 0:
            w.conv_t_kernel = put("ctk", p["short_conv_temporal"]["kernel"])
            w.conv_t_bias = put("ctb", p["short_conv_temporal"]["bias"])
        w.kernel = put("kernel", p["kernel"])
        names = ("delta_proj", "B_proj", "C_proj")
        if mod.gate_type == "factored":
            for g, n in enumerate(names):
                w.gate_kernel[2 * g] = put(f"g{g}hk", p[f"{n}_h"]["kernel"])
                w.gate_bias[2 * g] = put(f"g{g}hb", p[f"{n}_h"]["bias"])
                w.gate_kernel[2 * g + 1] = put(f"g{g}wk", p[f"{n}_w"]["kernel"])
                w.gate_bias[2 * g + 1] = put(f"g{g}wb", p[f"{n}_w"]["bias"])
        else:
            for g, n in enumerate(names):
                w.gate_kernel[g] = put(f"g{g}k", p[n]["kernel"])
                w.gate_bias[g] = put(f"g{g}b", p[n]["bias"])
        w.out_proj_kernel = put("opk", p["out_proj"]["kernel"])
        w.out_proj_bias = put("opb", p["out_proj"]["bias"])
        self.w = w
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}

    # plan per (T,H,W): K_hat and RoPE tables
    def plan(self, d: GatedDesc) -> torch.Tensor:
        key = (d.T, d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_gated_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError(
                    f"GatedCSSM: no CUDA kernel for shape/fields {tuple(getattr(d, f[0]) for f in d._fields_)}")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_gated_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                              _stream_ptr(self.device)), "cssm_gated_plan_init")
            self._plans[key] = pl
        return pl

    def desc(self, shape) -> GatedDesc:
        return self.mod._desc(shape)

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x)
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        n = self.L.cssm_gated_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        y = torch.empty_like(x) if out is None else out
        check(self.L.cssm_gated_forward(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                        y.data_ptr(), ws.data_ptr(), n, _stream_ptr(self.device)),
              "cssm_gated_forward")
        return y

    # ---- stage-level access (tests, profiling) ----
    def workspace_layout(self, d: GatedDesc) -> GatedWsLayout:
        l = GatedWsLayout()
        check(self.L.cssm_gated_workspace_layout(C.byref(d), C.byref(l)), "workspace_layout")
        return l

    def stages(self, x: torch.Tensor, upto: str = "out_proj"):
        """Runs the block stage by stage and returns the views of the workspace:
        xz (B*T, 2C, H, W), ctx_sum (B*T, C), gate_maps (B*T, H*Wf, 4) and y."""
        _require_cuda(x)
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        l = self.workspace_layout(d)
        ws = self.buf.get("ws", l.total)
        base = ws.data_ptr()
        st = _stream_ptr(self.device)
        B, T, H, W, Cc = x.shape
        Wf = W // 2 + 1
        f32 = ws.view(torch.float32)
        xz = f32[l.xz_planar // 4: l.xz_planar // 4 + B * T * 2 * Cc * H * W].view(B * T, 2 * Cc, H, W)
        ctx = f32[l.ctx_sum // 4: l.ctx_sum // 4 + B * T * Cc].view(B * T, Cc)
        gm = f32[l.gate_maps // 4: l.gate_maps // 4 + B * T * H * Wf * 4].view(B * T, H * Wf, 4)
        y = torch.empty_like(x)
        out = {"xz": xz, "ctx_sum": ctx, "gate_maps": gm, "y": y}
        order = ["in_proj", "short_conv", "gates", "spectral", "out_proj"]
        calls = {
            "in_proj": lambda: self.L.cssm_gated_in_proj(C.byref(d), C.byref(self.w), pl.data_ptr(),
                                                         x.data_ptr(), base + l.xz_planar, st),
            "short_conv": lambda: self.L.cssm_gated_short_conv(C.byref(d), C.byref(self.w),
                                                               base + l.xz_planar, base + l.ctx_sum, st),
            "gates": lambda: self.L.cssm_gated_gates(C.byref(d), C.byref(self.w), base + l.ctx_sum,
                                                     base + l.gate_maps, st),
            "spectral": lambda: self.L.cssm_gated_spectral(C.byref(d), pl.data_ptr(),
                                                           base + l.gate_maps, base + l.xz_planar, st),
            "out_proj": lambda: self.L.cssm_gated_out_proj(C.byref(d), C.byref(self.w),
                                                           base + l.xz_planar, y.data_ptr(), st),
        }
        for name in order:
            check(calls[name](), f"cssm_gated_{name}")
            if name == upto:
                break
        return out
