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


def _require_cuda(x, allow_bf16=False):
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("x must be a CUDA torch.Tensor (use forward_host for host arrays); "
                        "cssm_b200 has no CPU path")
    if x.dtype != torch.float32 and not (allow_bf16 and x.dtype == torch.bfloat16):
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
            _require_cuda(x, allow_bf16=True)
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

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 last_frame_only: bool = False, bf16_output: bool = False) -> torch.Tensor:
        """y = block(x).  With last_frame_only=True returns block(x)[:, -1] of shape (B,H,W,C)
        without computing the earlier output frames (for callers that read only the final
        frame, as SimpleCSSM with frame_readout='last' and CSSMSHViTBlock do).  A bfloat16 x
        (the SHViT mixers run in a bf16 model) is widened to fp32 and the result is float32, as
        Flax promotion gives with the block's fp32 parameters; bf16_output=True rounds it to
        bfloat16 instead."""
        _require_cuda(x, allow_bf16=True)
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        if x.dtype == torch.bfloat16:
            if last_frame_only:
                raise NotImplementedError("GatedCSSM: last_frame_only with bfloat16 activations")
            n = self.L.cssm_gated_bf16_workspace_bytes(C.byref(d))
            ws = self.buf.get("ws", n)
            odt = torch.bfloat16 if bf16_output else torch.float32
            y = torch.empty(x.shape, dtype=odt, device=x.device) if out is None else out
            check(self.L.cssm_gated_forward_bf16(C.byref(d), C.byref(self.w), pl.data_ptr(),
                                                 x.data_ptr(), y.data_ptr(), 1 if bf16_output else 0,
                                                 ws.data_ptr(), n, _stream_ptr(self.device)),
                  "cssm_gated_forward_bf16")
            return y
        n = self.L.cssm_gated_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        if last_frame_only:
            B, T, H, W, Cc = x.shape
            y = torch.empty((B, H, W, Cc), dtype=x.dtype, device=x.device) if out is None else out
            fn, what = self.L.cssm_gated_forward_last, "cssm_gated_forward_last"
        else:
            y = torch.empty_like(x) if out is None else out
            fn, what = self.L.cssm_gated_forward, "cssm_gated_forward"
        check(fn(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(), y.data_ptr(),
                 ws.data_ptr(), n, _stream_ptr(self.device)), what)
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


# ============================================================================== GDN
@dataclass
class GatedDeltaNetCSSM:
    """Gated DeltaNet spectral mixer (reference: GatedDeltaNetCSSM,
    src/models/cssm.py:4264-5141).  Same fields and defaults as the Flax dataclass; fields the
    d_k x d_k log-space path of the reference never reads (block_size, ssd_chunk_size,
    learned_init, scan_mode, use_complex32/16 with use_log=True) are accepted and have no
    effect here either."""
    channels: int
    delta_key_dim: int = 2
    kernel_size: int = 11
    rope_mode: str = "none"
    rope_base: float = 10000.0
    spectral_rho: float = 0.999
    position_independent_gates: bool = False
    block_size: int = 1
    gate_type: str = "channel"
    use_goom: bool = True
    use_log: bool = True
    use_complex32: bool = False
    use_complex16: bool = False
    scan_mode: str = "associative"
    ssd_chunk_size: int = 8
    learned_init: bool = False
    short_conv_size: int = 4
    output_norm: str = "rms"
    use_input_gates: bool = True
    output_gate_act: str = "silu"
    use_spectral_l2_norm: bool = True
    qkv_conv_size: int = 1
    qkv_conv_separable: bool = True
    cross_freq_conv_size: int = 0
    no_spectral_clamp: bool = False
    int_attention_mode: str = "none"
    attn_kernel_size: int = 7
    int_attn_dim: int = 16
    static_image_fast_path: bool = False
    num_timesteps: int = 0
    ssl_proj_dim: int = 0
    gate_proj_bias_init: float = 0.0
    name: Optional[str] = None
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    GATES = ("alpha", "beta", "B_k", "B_v")

    def param_shapes(self, H: int, W: int) -> Dict[str, Any]:
        Cc, Wf = self.channels, W // 2 + 1
        nh = Cc // self.delta_key_dim
        s: Dict[str, Any] = {
            "kernel": (nh, self.kernel_size, self.kernel_size),
            "qkv_proj": {"kernel": (Cc, 3 * Cc), "bias": (3 * Cc,)},
            "gate_proj": {"kernel": (Cc, Cc), "bias": (Cc,)},
            "output_proj": {"kernel": (Cc, Cc), "bias": (Cc,)},
        }
        if self.output_norm == "rms":
            s["rms_scale"] = (Cc,)
        if self.qkv_conv_size > 1:
            k = self.qkv_conv_size
            s["qkv_dw"] = {"kernel": (k, k, 1, Cc), "bias": (Cc,)}
        if self.short_conv_size > 0:
            for n in ("short_conv_q", "short_conv_k", "short_conv_v"):
                s[n] = {"kernel": (self.short_conv_size, 1, Cc), "bias": (Cc,)}
        gates = self.GATES if self.use_input_gates else self.GATES[:2]
        for n in gates:
            wd = W if n.startswith("B_") else Wf
            if self.gate_type == "factored":
                s[f"{n}_h"] = {"kernel": (Cc, H), "bias": (H,)}
                s[f"{n}_w"] = {"kernel": (Cc, wd), "bias": (wd,)}
            elif self.gate_type == "channel":
                # per-head scalars for alpha, beta; per-pixel 1x1 convs for B_k, B_v (cssm.py:4800-4810)
                s[n] = ({"kernel": (1, 1, Cc, Cc), "bias": (Cc,)} if n.startswith("B_")
                        else {"kernel": (Cc, nh), "bias": (nh,)})
            elif self.gate_type == "scalar":
                s[n] = {"kernel": (Cc, 1), "bias": (1,)}
            else:
                s[n] = {"kernel": (Cc, H * wd), "bias": (H * wd,)}
        return s

    def init(self, seed: int, x_shape, bias_scale: float = 0.0) -> Dict[str, Any]:
        _, _, H, W, Cc = x_shape
        rng = np.random.default_rng(seed)
        out: Dict[str, Any] = {}
        for k, v in self.param_shapes(H, W).items():
            if isinstance(v, dict):
                kern = v["kernel"]
                fan_in = kern[0] * kern[1] if k == "qkv_dw" else (kern[2] if len(kern) == 4 else kern[0])
                b = bias_scale * rng.standard_normal(v["bias"])
                if k == "gate_proj":
                    b = b + self.gate_proj_bias_init
                out[k] = {"kernel": (rng.standard_normal(kern) / np.sqrt(fan_in)).astype(np.float32),
                          "bias": b.astype(np.float32)}
            elif k == "rms_scale":
                out[k] = np.ones(v, np.float32)
            else:   # spectral kernel, xavier-normal over (n_h, ks, ks)
                std = np.sqrt(2.0 / (2 * v[0] * v[1]))
                out[k] = (std * rng.standard_normal(v)).astype(np.float32)
        return {"params": out}

    def _check_fields(self):
        bad = []
        if self.gate_type not in _lib.GDN_GATE_TYPES:
            bad.append(f"gate_type={self.gate_type!r} (have 'factored', 'dense', 'channel', 'scalar')")
        if not (self.use_log and self.use_goom) and (self.use_complex32 or self.use_complex16):
            bad.append("bf16/fp8 split-precision scans")
        if self.position_independent_gates:
            bad.append("position_independent_gates")
        if self.rope_mode not in ROPE_MODES:
            bad.append(f"rope_mode={self.rope_mode!r}")
        if self.output_norm not in ("rms", "none"):
            bad.append(f"output_norm={self.output_norm!r}")
        if self.qkv_conv_size > 1 and not self.qkv_conv_separable:
            bad.append("non-separable qkv conv")
        if self.cross_freq_conv_size or self.int_attention_mode != "none" or self.ssl_proj_dim:
            bad.append("cross_freq_conv / int_attention / ssl_proj")
        if self.static_image_fast_path:
            # the reference asserts these (cssm.py:4354-4370)
            if self.short_conv_size != 0 or self.use_input_gates or self.rope_mode != "none":
                raise AssertionError("static_image_fast_path requires short_conv_size=0, "
                                     "use_input_gates=False, rope_mode='none'")
            if self.num_timesteps <= 0:
                raise AssertionError("static_image_fast_path requires num_timesteps > 0")
            if self.output_norm == "layer":
                bad.append("output_norm='layer'")
            if self.gate_type in ("channel", "scalar"):
                bad.append(f"static_image_fast_path with gate_type={self.gate_type!r}")
        if self.output_gate_act not in ("silu", "sigmoid"):
            bad.append(f"output_gate_act={self.output_gate_act!r}")
        if self.delta_key_dim > 4:
            bad.append("delta_key_dim > 4")
        if bad:
            raise NotImplementedError("GatedDeltaNetCSSM: no CUDA kernel for " + "; ".join(bad))

    def _desc(self, shape) -> GdnDesc:
        B, T, H, W, Cc = shape
        if Cc != self.channels:
            raise ValueError(f"x has {Cc} channels, module has {self.channels}")
        if Cc % self.delta_key_dim:
            raise AssertionError(f"channels={Cc} must be divisible by delta_key_dim={self.delta_key_dim}")
        return GdnDesc(B, T, H, W, Cc, self.delta_key_dim, self.kernel_size,
                       ROPE_MODES[self.rope_mode], float(self.rope_base), float(self.spectral_rho),
                       _lib.GDN_GATE_TYPES[self.gate_type], self.short_conv_size,
                       1 if self.output_norm == "rms" else 0, int(self.use_input_gates),
                       0 if self.output_gate_act == "silu" else 1, int(self.use_spectral_l2_norm),
                       self.qkv_conv_size, int(self.no_spectral_clamp))

    def bind(self, variables, device="cuda") -> "BoundGdn":
        self._check_fields()
        return BoundGdn(self, variables["params"] if "params" in variables else variables,
                        torch.device(device))

    def apply(self, variables, x, injected_qkv_spatial=None):
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            _require_cuda(x)
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


class BoundGdn:
    def __init__(self, mod: GatedDeltaNetCSSM, p, device):
        self.mod, self.device, self.variables_ref = mod, device, None
        self.L = _lib.lib()
        self.t: Dict[str, torch.Tensor] = {}

        def put(name, arr):
            self.t[name] = _dev_f32(arr, device)
            return self.t[name].data_ptr()

        w = GdnWeights()
        w.kernel = put("kernel", p["kernel"])
        if mod.qkv_conv_size > 1:
            w.qkv_dw_kernel = put("dwk", p["qkv_dw"]["kernel"])
            w.qkv_dw_bias = put("dwb", p["qkv_dw"]["bias"])
        w.qkv_proj_kernel = put("qk", p["qkv_proj"]["kernel"])
        w.qkv_proj_bias = put("qb", p["qkv_proj"]["bias"])
        if mod.short_conv_size > 0:
            for i, n in enumerate(("short_conv_q", "short_conv_k", "short_conv_v")):
                w.conv_t_kernel[i] = put(f"ct{i}k", p[n]["kernel"])
                w.conv_t_bias[i] = put(f"ct{i}b", p[n]["bias"])
        gates = mod.GATES if mod.use_input_gates else mod.GATES[:2]
        for g, n in enumerate(gates):
            if mod.gate_type == "factored":
                w.gate_kernel[2 * g] = put(f"g{g}hk", p[f"{n}_h"]["kernel"])
                w.gate_bias[2 * g] = put(f"g{g}hb", p[f"{n}_h"]["bias"])
                w.gate_kernel[2 * g + 1] = put(f"g{g}wk", p[f"{n}_w"]["kernel"])
                w.gate_bias[2 * g + 1] = put(f"g{g}wb", p[f"{n}_w"]["bias"])
            else:
                w.gate_kernel[g] = put(f"g{g}k", p[n]["kernel"])
                w.gate_bias[g] = put(f"g{g}b", p[n]["bias"])
        w.gate_proj_kernel = put("gpk", p["gate_proj"]["kernel"])
        w.gate_proj_bias = put("gpb", p["gate_proj"]["bias"])
        if mod.output_norm == "rms":
            w.rms_scale = put("rms", p["rms_scale"])
        w.output_proj_kernel = put("opk", p["output_proj"]["kernel"])
        w.output_proj_bias = put("opb", p["output_proj"]["bias"])
        self.w = w
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}

    def desc(self, shape) -> GdnDesc:
        return self.mod._desc(shape)

    def plan(self, d: GdnDesc) -> torch.Tensor:
        key = (d.T, d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_gdn_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError(
                    f"GatedDeltaNetCSSM: no CUDA kernel for {tuple(getattr(d, f[0]) for f in d._fields_)}")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_gdn_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                            _stream_ptr(self.device)), "cssm_gdn_plan_init")
            self._plans[key] = pl
        return pl

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 last_frame_only: bool = False) -> torch.Tensor:
        """y = block(x).  With last_frame_only=True returns block(x)[:, -1] of shape (B,H,W,C)
        (for callers with a last-frame readout): the readout, inverse transforms and output
        projections of the earlier frames are not computed.  A 4-D x (B,H,W,C) takes the
        static-image fast path when the module was built with static_image_fast_path=True
        (T = num_timesteps gate steps, bf16 carry, final readout; returns (B,H,W,C))."""
        _require_cuda(x)
        x = x.contiguous()
        if x.dim() == 4:
            if not self.mod.static_image_fast_path:
                raise ValueError("GatedDeltaNetCSSM: a 4-D input needs static_image_fast_path=True")
            B, H, W, Cc = x.shape
            d = self.desc((B, self.mod.num_timesteps, H, W, Cc))
            pl = self.plan(d)
            n = self.L.cssm_gdn_workspace_bytes(C.byref(d))
            ws = self.buf.get("ws", n)
            y = torch.empty_like(x) if out is None else out
            check(self.L.cssm_gdn_forward_static_image(C.byref(d), C.byref(self.w), pl.data_ptr(),
                                                       x.data_ptr(), y.data_ptr(), ws.data_ptr(), n,
                                                       _stream_ptr(self.device)),
                  "cssm_gdn_forward_static_image")
            return y
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        n = self.L.cssm_gdn_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        if last_frame_only:
            B, T, H, W, Cc = x.shape
            y = torch.empty((B, H, W, Cc), dtype=x.dtype, device=x.device) if out is None else out
            fn, what = self.L.cssm_gdn_forward_last, "cssm_gdn_forward_last"
        else:
            y = torch.empty_like(x) if out is None else out
            fn, what = self.L.cssm_gdn_forward, "cssm_gdn_forward"
        check(fn(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(), y.data_ptr(),
                 ws.data_ptr(), n, _stream_ptr(self.device)), what)
        return y


# ========================================================================== no gate
@dataclass
class NoGateCSSM:
    """Ungated spectral block (reference: NoGateCSSM, src/models/cssm.py:6101-6175):
    rfft2(x) -> S_t = K_hat S_{t-1} + X_hat_t -> irfft2 -> out_proj, returned minus x.
    Fields the reference accepts for interface compatibility and never reads
    (rope_mode, short_conv_*, block_size, gate_type, ...) are accepted here too."""
    channels: int
    kernel_size: int = 11
    spectral_rho: float = 0.999
    rope_mode: str = "none"
    rope_base: float = 10000.0
    short_conv_size: int = 4
    short_conv_spatial_size: int = 0
    block_size: int = 1
    position_independent_gates: bool = False
    gate_type: str = "dense"
    name: Optional[str] = None
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    def param_shapes(self, H: int, W: int) -> Dict[str, Any]:
        Cc = self.channels
        return {"kernel": (Cc, self.kernel_size, self.kernel_size),
                "out_proj": {"kernel": (Cc, Cc), "bias": (Cc,)}}

    def init(self, seed: int, x_shape, bias_scale: float = 0.0) -> Dict[str, Any]:
        rng = np.random.default_rng(seed)
        Cc = self.channels
        return {"params": {
            "kernel": (0.02 * rng.standard_normal((Cc, self.kernel_size, self.kernel_size))).astype(np.float32),
            "out_proj": {"kernel": (rng.standard_normal((Cc, Cc)) / np.sqrt(Cc)).astype(np.float32),
                         "bias": (bias_scale * rng.standard_normal(Cc)).astype(np.float32)}}}

    def bind(self, variables, device="cuda") -> "BoundNoGate":
        return BoundNoGate(self, variables["params"] if "params" in variables else variables,
                           torch.device(device))

    def apply(self, variables, x, injected_qkv_spatial=None):
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            _require_cuda(x)
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


class BoundNoGate:
    """A NoGateCSSM with its weights resident on one GPU and its plan cached per (H, W)."""

    def __init__(self, mod: NoGateCSSM, params, device):
        self.mod, self.device, self.variables_ref = mod, device, None
        self.L = _lib.lib()
        self.t = {"k": _dev_f32(params["kernel"], device),
                  "ok": _dev_f32(params["out_proj"]["kernel"], device),
                  "ob": _dev_f32(params["out_proj"]["bias"], device)}
        self.w = _lib.NoGateWeights(self.t["k"].data_ptr(), self.t["ok"].data_ptr(), self.t["ob"].data_ptr())
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}

    def desc(self, shape):
        B, T, H, W, Cc = shape
        if Cc != self.mod.channels:
            raise ValueError(f"x has {Cc} channels, module has {self.mod.channels}")
        return _lib.NoGateDesc(B, T, H, W, Cc, self.mod.kernel_size, float(self.mod.spectral_rho))

    def plan(self, d) -> torch.Tensor:
        """The weight-only plan (K_hat) for descriptor d, built once per plane size."""
        key = (d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_nogate_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError("NoGateCSSM: no CUDA kernel for this shape")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_nogate_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                               _stream_ptr(self.device)), "cssm_nogate_plan_init")
            self._plans[key] = pl
        return pl

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x)
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        n = self.L.cssm_nogate_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        y = torch.empty_like(x) if out is None else out
        check(self.L.cssm_nogate_forward(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                         y.data_ptr(), ws.data_ptr(), n, _stream_ptr(self.device)),
              "cssm_nogate_forward")
        return y


# ============================================================================ additive (1 state)
@dataclass
class AdditiveCSSM:
    """Single-state path of the reference's AdditiveCSSM (src/models/cssm.py:2961-3359,
    3580-3626): x_proj -> rfft2 -> h_t = (d_X K_hat) h_{t-1} + B_X X_hat_t -> C_gate h_t ->
    irfft2 -> output_proj.  Field names and defaults are the reference's; only
    single_state=True with gate_type 'dense', 'factored' or 'channel' (d_X per channel, B_X and
    C_gate per-pixel 1x1-conv maps applied in the spatial domain) has a CUDA path, everything else
    raises NotImplementedError (no fallback)."""
    channels: int
    kernel_size: int = 11
    rope_mode: str = "none"
    rope_base: float = 10000.0
    spectral_rho: float = 0.999
    position_independent_gates: bool = False
    block_size: int = 1
    no_k_state: bool = False
    single_state: bool = False
    use_goom: bool = True
    gate_type: str = "dense"
    learned_init: bool = False
    use_complex32: bool = False
    use_complex16: bool = False
    use_ssd: bool = False
    scan_mode: str = "associative"
    ssd_chunk_size: int = 8
    use_delta: bool = False
    l2_norm_qk: bool = False
    name: Optional[str] = None
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    GATES = ("d_X", "B_X", "C_gate")

    def _check(self):
        if not self.single_state:
            raise NotImplementedError("AdditiveCSSM: only single_state=True has a CUDA path "
                                      "(the 2- and 3-state triangular scans are not built)")
        if self.gate_type not in ("dense", "factored", "channel"):
            raise NotImplementedError(f"AdditiveCSSM: gate_type {self.gate_type!r} not built "
                                      "(supported: 'dense', 'factored', 'channel')")
        if self.rope_mode not in ROPE_MODES:
            raise NotImplementedError(f"AdditiveCSSM: rope_mode {self.rope_mode!r} not built")
        if self.position_independent_gates or self.learned_init:
            raise NotImplementedError("AdditiveCSSM: position_independent_gates / learned_init not built")
        if self.use_complex32 or self.use_complex16:
            raise NotImplementedError("AdditiveCSSM: the bf16 / fp8 linear-split scans are not built")
        if self.scan_mode not in ("associative", "ssd", "quadratic", "pallas"):
            raise ValueError(f"AdditiveCSSM: unknown scan_mode {self.scan_mode!r}")
        if not self.use_goom and self._floor():
            raise NotImplementedError("AdditiveCSSM: use_goom=False with the associative scan not built")

    def _floor(self) -> int:
        """1 when the reference runs the log-space scan (its 1e-7 magnitude floors apply)."""
        return 1 if (self.scan_mode == "associative" and not self.use_ssd) else 0

    def param_shapes(self, H: int, W: int) -> Dict[str, Any]:
        Cc, Wf = self.channels, W // 2 + 1
        p = {"kernel": (Cc, self.kernel_size, self.kernel_size),
             "x_proj": {"kernel": (Cc, Cc), "bias": (Cc,)},
             "output_proj": {"kernel": (Cc, Cc), "bias": (Cc,)}}
        for n in self.GATES:
            if self.gate_type == "factored":
                p[f"{n}_h"] = {"kernel": (Cc, H), "bias": (H,)}
                p[f"{n}_w"] = {"kernel": (Cc, Wf), "bias": (Wf,)}
            elif self.gate_type == "channel":
                # d_X: Dense(C); B_X, C_gate: 1x1 convs (cssm.py:3168-3178)
                p[n] = {"kernel": (Cc, Cc) if n == "d_X" else (1, 1, Cc, Cc), "bias": (Cc,)}
            else:
                p[n] = {"kernel": (Cc, H * Wf), "bias": (H * Wf,)}
        return p

    def init(self, seed: int, x_shape, bias_scale: float = 0.0) -> Dict[str, Any]:
        """Seeded stand-ins for the Flax initialisers, in the reference's parameter tree."""
        self._check()
        _, _, H, W, _ = x_shape
        rng = np.random.default_rng(seed)

        def fill(shape_tree, name=""):
            if isinstance(shape_tree, dict):
                return {k: fill(v, k) for k, v in shape_tree.items()}
            if name == "bias":
                return (bias_scale * rng.standard_normal(shape_tree)).astype(np.float32)
            fan_in = (shape_tree[0] if len(shape_tree) == 2 else
                      shape_tree[2] if len(shape_tree) == 4 else 2 * self.kernel_size * self.channels / 2)
            return (rng.standard_normal(shape_tree) / np.sqrt(fan_in)).astype(np.float32)
        return {"params": fill(self.param_shapes(H, W))}

    def bind(self, variables, device="cuda") -> "BoundAdditive":
        self._check()
        return BoundAdditive(self, variables["params"] if "params" in variables else variables,
                             torch.device(device))

    def apply(self, variables, x, injected_qkv_spatial=None):
        if injected_qkv_spatial is not None:
            raise NotImplementedError("AdditiveCSSM: injected_qkv_spatial not built")
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            _require_cuda(x)
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


class BoundAdditive:
    """A single-state AdditiveCSSM with its weights on one GPU and its plan cached per (T, H, W)."""

    def __init__(self, mod: AdditiveCSSM, params, device):
        self.mod, self.device, self.variables_ref = mod, device, None
        self.L = _lib.lib()
        self.params = params
        self.t: Dict[str, torch.Tensor] = {}
        w = _lib.AdditiveWeights()
        w.kernel = self._put("kernel", params["kernel"])
        w.x_proj_kernel = self._put("xk", params["x_proj"]["kernel"])
        w.x_proj_bias = self._put("xb", params["x_proj"]["bias"])
        w.output_proj_kernel = self._put("ok", params["output_proj"]["kernel"])
        w.output_proj_bias = self._put("ob", params["output_proj"]["bias"])
        names = ([f"{n}_{s}" for n in mod.GATES for s in ("h", "w")]
                 if mod.gate_type == "factored" else list(mod.GATES))
        for i, n in enumerate(names):
            if n not in params:
                raise KeyError(f"AdditiveCSSM: parameter {n!r} missing (gate_type={mod.gate_type!r})")
            w.gate_kernel[i] = self._put(f"gk{i}", params[n]["kernel"])
            w.gate_bias[i] = self._put(f"gb{i}", params[n]["bias"])
        self.w = w
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}

    def _put(self, key, arr) -> int:
        self.t[key] = _dev_f32(arr, self.device)
        return self.t[key].data_ptr()

    def desc(self, shape):
        B, T, H, W, Cc = shape
        m = self.mod
        if Cc != m.channels:
            raise ValueError(f"x has {Cc} channels, module has {m.channels}")
        Wf = W // 2 + 1
        gshape = tuple(self.t["gk0"].shape)
        want = {"factored": (Cc, H), "channel": (Cc, Cc)}.get(m.gate_type, (Cc, H * Wf))
        if gshape != want:
            raise ValueError(f"AdditiveCSSM: gate weights {gshape} were made for another plane size "
                             f"(this input needs {want})")
        return _lib.AdditiveDesc(B, T, H, W, Cc, m.kernel_size, ROPE_MODES[m.rope_mode],
                                 float(m.rope_base), float(m.spectral_rho),
                                 _lib.DELTANET_GATE_TYPES[m.gate_type], 1, m._floor())

    def plan(self, d) -> torch.Tensor:
        """The weight-only plan (kernel spectrum, RoPE tables, temporal code) for descriptor d."""
        key = (d.T, d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_additive_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError("AdditiveCSSM: no CUDA kernel for this shape")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_additive_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                                 _stream_ptr(self.device)), "cssm_additive_plan_init")
            self._plans[key] = pl
        return pl

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x)
        if x.dim() != 5:
            raise ValueError("AdditiveCSSM expects (B,T,H,W,C)")
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        n = self.L.cssm_additive_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        y = torch.empty_like(x) if out is None else out
        check(self.L.cssm_additive_forward(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                           y.data_ptr(), ws.data_ptr(), n, _stream_ptr(self.device)),
              "cssm_additive_forward")
        return y


# ============================================================================ DeltaNet (scalar)
@dataclass
class DeltaNetCSSM:
    """Scalar spectral delta rule (reference: DeltaNetCSSM, src/models/cssm.py:3628-3930).
    Field names and defaults are the reference's.  The CUDA path covers gate_type 'channel' (the
    default: per-channel decay scalars, 1x1-conv spatial I/O gates), 'dense' and 'factored'; the
    other gate types raise NotImplementedError, as do learned_init, position_independent_gates
    and the bf16 / fp8 split scans (no fallback)."""
    channels: int
    kernel_size: int = 11
    rope_mode: str = "none"
    rope_base: float = 10000.0
    spectral_rho: float = 0.999
    position_independent_gates: bool = False
    block_size: int = 1
    gate_type: str = "channel"
    use_goom: bool = True
    use_complex32: bool = False
    use_complex16: bool = False
    scan_mode: str = "associative"
    ssd_chunk_size: int = 8
    learned_init: bool = False
    name: Optional[str] = None
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    GATES = ("alpha", "beta", "B_k", "B_v", "C_gate")

    def _check(self):
        if self.gate_type not in _lib.DELTANET_GATE_TYPES:
            raise NotImplementedError(f"DeltaNetCSSM: gate_type {self.gate_type!r} not built "
                                      "(supported: 'channel', 'dense', 'factored')")
        if self.rope_mode not in ROPE_MODES:
            raise NotImplementedError(f"DeltaNetCSSM: rope_mode {self.rope_mode!r} not built")
        if self.position_independent_gates or self.learned_init:
            raise NotImplementedError("DeltaNetCSSM: position_independent_gates / learned_init not built")
        if self.use_complex32 or self.use_complex16:
            raise NotImplementedError("DeltaNetCSSM: the bf16 / fp8 linear-split scans are not built")
        if self.scan_mode not in ("associative", "ssd", "quadratic", "pallas"):
            raise ValueError(f"DeltaNetCSSM: unknown scan_mode {self.scan_mode!r}")
        if not self.use_goom and self._floor():
            raise NotImplementedError("DeltaNetCSSM: use_goom=False with the associative scan not built")

    def _floor(self) -> int:
        return 1 if self.scan_mode == "associative" else 0

    def param_shapes(self, H: int, W: int) -> Dict[str, Any]:
        Cc, Wf = self.channels, W // 2 + 1
        p = {"kernel": (Cc, self.kernel_size, self.kernel_size),
             "qkv_proj": {"kernel": (Cc, 3 * Cc), "bias": (3 * Cc,)},
             "output_proj": {"kernel": (Cc, Cc), "bias": (Cc,)}}
        for n in self.GATES:
            if self.gate_type == "channel":
                # alpha, beta: Dense(C); B_k, B_v, C_gate: Conv 1x1 (HWIO)
                p[n] = {"kernel": (Cc, Cc) if n in ("alpha", "beta") else (1, 1, Cc, Cc), "bias": (Cc,)}
            elif self.gate_type == "factored":
                p[f"{n}_h"] = {"kernel": (Cc, H), "bias": (H,)}
                p[f"{n}_w"] = {"kernel": (Cc, Wf), "bias": (Wf,)}
            else:
                p[n] = {"kernel": (Cc, H * Wf), "bias": (H * Wf,)}
        return p

    def init(self, seed: int, x_shape, bias_scale: float = 0.0) -> Dict[str, Any]:
        """Seeded stand-ins for the Flax initialisers, in the reference's parameter tree."""
        self._check()
        _, _, H, W, _ = x_shape
        rng = np.random.default_rng(seed)

        def fill(shape_tree, name=""):
            if isinstance(shape_tree, dict):
                return {k: fill(v, k) for k, v in shape_tree.items()}
            if name == "bias":
                return (bias_scale * rng.standard_normal(shape_tree)).astype(np.float32)
            fan_in = (shape_tree[0] if len(shape_tree) == 2 else
                      self.channels if len(shape_tree) == 4 else self.kernel_size * self.channels)
            return (rng.standard_normal(shape_tree) / np.sqrt(fan_in)).astype(np.float32)
        return {"params": fill(self.param_shapes(H, W))}

    def bind(self, variables, device="cuda") -> "BoundDeltaNet":
        self._check()
        return BoundDeltaNet(self, variables["params"] if "params" in variables else variables,
                             torch.device(device))

    def apply(self, variables, x, injected_qkv_spatial=None):
        # the reference ignores injected_qkv_spatial in this block (cssm.py:3675-3676)
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            _require_cuda(x)
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


class BoundDeltaNet:
    """A DeltaNetCSSM with its weights on one GPU and its plan cached per (T, H, W)."""

    def __init__(self, mod: DeltaNetCSSM, params, device):
        self.mod, self.device, self.variables_ref = mod, device, None
        self.L = _lib.lib()
        self.t: Dict[str, torch.Tensor] = {}
        w = _lib.DeltaNetWeights()
        w.kernel = self._put("kernel", params["kernel"])
        w.qkv_proj_kernel = self._put("qk", params["qkv_proj"]["kernel"])
        w.qkv_proj_bias = self._put("qb", params["qkv_proj"]["bias"])
        w.output_proj_kernel = self._put("ok", params["output_proj"]["kernel"])
        w.output_proj_bias = self._put("ob", params["output_proj"]["bias"])
        names = ([f"{n}_{s}" for n in mod.GATES for s in ("h", "w")]
                 if mod.gate_type == "factored" else list(mod.GATES))
        for i, n in enumerate(names):
            if n not in params:
                raise KeyError(f"DeltaNetCSSM: parameter {n!r} missing (gate_type={mod.gate_type!r})")
            w.gate_kernel[i] = self._put(f"gk{i}", params[n]["kernel"])
            w.gate_bias[i] = self._put(f"gb{i}", params[n]["bias"])
        self.w = w
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}

    def _put(self, key, arr) -> int:
        self.t[key] = _dev_f32(arr, self.device)
        return self.t[key].data_ptr()

    def desc(self, shape):
        B, T, H, W, Cc = shape
        m = self.mod
        if Cc != m.channels:
            raise ValueError(f"x has {Cc} channels, module has {m.channels}")
        Wf = W // 2 + 1
        gshape = tuple(self.t["gk0"].shape)
        want = {"factored": (Cc, H), "dense": (Cc, H * Wf), "channel": (Cc, Cc)}[m.gate_type]
        if gshape != want:
            raise ValueError(f"DeltaNetCSSM: gate weights {gshape} were made for another plane size "
                             f"(this input needs {want})")
        return _lib.DeltaNetDesc(B, T, H, W, Cc, m.kernel_size, ROPE_MODES[m.rope_mode],
                                 float(m.rope_base), float(m.spectral_rho),
                                 _lib.DELTANET_GATE_TYPES[m.gate_type], m._floor())

    def plan(self, d) -> torch.Tensor:
        """The weight-only plan (kernel spectrum, RoPE tables, temporal code) for descriptor d."""
        key = (d.T, d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_deltanet_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError("DeltaNetCSSM: no CUDA kernel for this shape")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_deltanet_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                                 _stream_ptr(self.device)), "cssm_deltanet_plan_init")
            self._plans[key] = pl
        return pl

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x)
        if x.dim() != 5:
            raise ValueError("DeltaNetCSSM expects (B,T,H,W,C)")
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        n = self.L.cssm_deltanet_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        y = torch.empty_like(x) if out is None else out
        check(self.L.cssm_deltanet_forward(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                           y.data_ptr(), ws.data_ptr(), n, _stream_ptr(self.device)),
              "cssm_deltanet_forward")
        return y
