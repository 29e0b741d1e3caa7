"""Host-side mirror of the reference's SimpleCSSM wrapper (src/models/simple_cssm.py:62-558)
for inference with ONE spectral block: stem -> x + block(x) -> last-frame readout -> logits.

Field names and defaults are the reference's.  Supported: depth 1; cssm_type 'gated' / 'gdn' /
'no_gate' / 'add_kqv_1' / 'deltanet' (CSSM_REGISTRY names, simple_cssm.py:21-60);
stem_mode 'default' (stem_layers x [conv3x3, softplus, LayerNorm, 2x2 max-pool]) and
'pathtracker' (conv1x1, softplus, LayerNorm); stem_norm_order 'post'; act_type 'softplus';
norm_type 'layer'; frame_readout 'last'; pool_type 'mean' / 'max'; readout_norm 'pre' / 'post';
pos_embed in the RoPE modes of the block or 'none'; embed_dim <= 64.  Everything else raises
NotImplementedError: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import numpy as np
import torch

from . import _lib
from ._lib import SIMPLE_LAST_FRAME_ONLY, SimpleDesc, SimpleWeights, check
from .modules import (AdditiveCSSM, DeltaNetCSSM, GatedCSSM, GatedDeltaNetCSSM, NoGateCSSM, _Buffers,
                      _dev_f32, _require_cuda, _stream_ptr)


@dataclass
class SimpleCSSM:
    num_classes: int = 2
    embed_dim: int = 32
    depth: int = 1
    cssm_type: str = "hgru_bi"
    kernel_size: int = 15
    block_size: int = 1
    frame_readout: str = "last"
    norm_type: str = "layer"
    stem_norm: str = ""
    body_norm: str = ""
    pos_embed: str = "spatiotemporal"
    act_type: str = "softplus"
    pool_type: str = "mean"
    seq_len: int = 8
    gate_type: str = "dense"
    n_register_tokens: int = 0
    stem_mode: str = "default"
    stem_layers: int = 2
    stem_norm_order: str = "post"
    readout_norm: str = "pre"
    short_conv_size: int = 4
    short_conv_spatial_size: int = 3
    output_norm: str = "rms"
    use_input_gates: bool = True
    output_gate_act: str = "silu"
    use_spectral_l2_norm: bool = True
    qkv_conv_size: int = 1
    qkv_conv_separable: bool = True
    delta_key_dim: int = 2
    no_spectral_clamp: bool = False
    use_goom: bool = True
    learned_init: bool = False
    use_complex32: bool = False
    use_complex16: bool = False
    use_ssd: bool = False
    scan_mode: str = "associative"
    ssd_chunk_size: int = 8
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    # -- the block this model wraps (simple_cssm.py:318-481) -----------------------------
    def block(self):
        rope = self.pos_embed if self.pos_embed in ("spatiotemporal", "spatial_only", "temporal", "mrope") else "none"
        if self.cssm_type == "gated":
            return GatedCSSM(channels=self.embed_dim, kernel_size=self.kernel_size, rope_mode=rope,
                             short_conv_spatial_size=self.short_conv_spatial_size,
                             short_conv_size=self.short_conv_size, gate_type=self.gate_type)
        if self.cssm_type == "gdn":
            return GatedDeltaNetCSSM(channels=self.embed_dim, kernel_size=self.kernel_size,
                                     rope_mode=rope, short_conv_size=self.short_conv_size,
                                     gate_type=self.gate_type, output_norm=self.output_norm,
                                     use_input_gates=self.use_input_gates,
                                     output_gate_act=self.output_gate_act,
                                     use_spectral_l2_norm=self.use_spectral_l2_norm,
                                     qkv_conv_size=self.qkv_conv_size,
                                     qkv_conv_separable=self.qkv_conv_separable,
                                     delta_key_dim=self.delta_key_dim,
                                     no_spectral_clamp=self.no_spectral_clamp)
        if self.cssm_type == "no_gate":                      # simple_cssm.py:344-347
            return NoGateCSSM(channels=self.embed_dim, kernel_size=self.kernel_size, rope_mode=rope,
                              block_size=self.block_size, short_conv_size=self.short_conv_size,
                              short_conv_spatial_size=self.short_conv_spatial_size)
        scan = dict(use_goom=self.use_goom, gate_type=self.gate_type, learned_init=self.learned_init,
                    use_complex32=self.use_complex32, use_complex16=self.use_complex16,
                    scan_mode=self.scan_mode, ssd_chunk_size=self.ssd_chunk_size)
        if self.cssm_type == "add_kqv_1":                    # simple_cssm.py:368-381
            return AdditiveCSSM(channels=self.embed_dim, kernel_size=self.kernel_size, rope_mode=rope,
                                block_size=self.block_size, single_state=True, use_ssd=self.use_ssd,
                                **scan)
        if self.cssm_type == "deltanet":                     # simple_cssm.py:385-393
            return DeltaNetCSSM(channels=self.embed_dim, kernel_size=self.kernel_size, rope_mode=rope,
                                block_size=self.block_size, **scan)
        raise NotImplementedError(f"SimpleCSSM: cssm_type={self.cssm_type!r} has no CUDA kernel "
                                  "(have 'gated', 'gdn', 'no_gate', 'add_kqv_1', 'deltanet')")

    def _check_fields(self):
        bad = []
        if self.depth != 1:
            bad.append(f"depth={self.depth}")
        if self.frame_readout != "last":
            bad.append(f"frame_readout={self.frame_readout!r}")
        if self.act_type != "softplus":
            bad.append(f"act_type={self.act_type!r}")
        for n in (self.norm_type, self.stem_norm or "layer", self.body_norm or "layer"):
            if n != "layer":
                bad.append(f"norm {n!r}")
        if self.stem_norm_order != "post":
            bad.append(f"stem_norm_order={self.stem_norm_order!r}")
        if self.stem_mode not in ("default", "pathtracker"):
            bad.append(f"stem_mode={self.stem_mode!r}")
        if self.pool_type not in ("mean", "max") or self.readout_norm not in ("pre", "post"):
            bad.append("pool_type / readout_norm")
        if self.pos_embed in ("learnable", "separate", "sinusoidal"):
            bad.append(f"pos_embed={self.pos_embed!r}")
        if self.n_register_tokens:
            bad.append("register tokens")
        if self.embed_dim > 64 or self.embed_dim % 4:
            bad.append(f"embed_dim={self.embed_dim}")
        if bad:
            raise NotImplementedError("SimpleCSSM: no CUDA kernel for " + "; ".join(bad))
        check_block = getattr(self.block(), "_check", None)     # field combinations of the block
        if check_block is not None:
            check_block()

    def feature_hw(self, Hin: int, Win: int):
        H, W = Hin, Win
        if self.stem_mode == "default":
            for _ in range(self.stem_layers):
                H, W = (H + 1) // 2, (W + 1) // 2
        return H, W

    def param_shapes(self, Hin: int, Win: int, Cin: int) -> Dict[str, Any]:
        E = self.embed_dim
        s: Dict[str, Any] = {}
        if self.stem_mode == "pathtracker":
            s["conv1"] = {"kernel": (1, 1, Cin, E), "bias": (E,)}
            s["norm1"] = {"scale": (E,), "bias": (E,)}
        else:
            ci = Cin
            for i in range(self.stem_layers):
                s[f"conv{i + 1}"] = {"kernel": (3, 3, ci, E), "bias": (E,)}
                s[f"norm{i + 1}"] = {"scale": (E,), "bias": (E,)}
                ci = E
        H, W = self.feature_hw(Hin, Win)
        s["cssm_0"] = self.block().param_shapes(H, W)
        s["norm_pre"] = {"scale": (E,), "bias": (E,)}
        s["norm_post"] = {"scale": (E,), "bias": (E,)}
        s["head"] = {"kernel": (E, self.num_classes), "bias": (self.num_classes,)}
        return s

    def init(self, seed: int, x_shape, bias_scale: float = 0.0) -> Dict[str, Any]:
        """Random-init variables {'params': tree} (NumPy-seeded stand-ins for the Flax
        initialisers).  x_shape: (B,H,W,Cin) or (B,T,H,W,Cin)."""
        Hin, Win, Cin = x_shape[-3:]
        rng = np.random.default_rng(seed)
        E = self.embed_dim
        H, W = self.feature_hw(Hin, Win)
        T = self.seq_len if len(x_shape) == 4 else x_shape[1]
        out: Dict[str, Any] = {}
        for k, v in self.param_shapes(Hin, Win, Cin).items():
            if k == "cssm_0":
                out[k] = self.block().init(seed + 1, (x_shape[0], T, H, W, E), bias_scale)["params"]
            elif "scale" in v:
                out[k] = {"scale": (1.0 + bias_scale * rng.standard_normal(v["scale"])).astype(np.float32),
                          "bias": (bias_scale * rng.standard_normal(v["bias"])).astype(np.float32)}
            else:
                kern = v["kernel"]
                fan_in = int(np.prod(kern[:-1]))
                out[k] = {"kernel": (rng.standard_normal(kern) / np.sqrt(fan_in)).astype(np.float32),
                          "bias": (bias_scale * rng.standard_normal(v["bias"])).astype(np.float32)}
        return {"params": out}

    def bind(self, variables, device="cuda") -> "BoundSimple":
        self._check_fields()
        return BoundSimple(self, variables["params"] if "params" in variables else variables,
                           torch.device(device))

    def apply(self, variables, x, training: bool = False):
        """Flax-style call: logits = model.apply({'params': tree}, x, training=False)."""
        if training:
            raise NotImplementedError("SimpleCSSM: inference only")
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            _require_cuda(x)
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


class BoundSimple:
    """A SimpleCSSM with its weights resident on one GPU."""

    def __init__(self, mod: SimpleCSSM, params, device):
        self.mod = mod
        self.device = device
        self.variables_ref = None
        self.L = _lib.lib()
        self.block = mod.block().bind(params["cssm_0"], device)
        self.t: Dict[str, torch.Tensor] = {}

        def put(name, arr):
            self.t[name] = _dev_f32(arr, device)
            return self.t[name].data_ptr()

        w = SimpleWeights()
        nl = 1 if mod.stem_mode == "pathtracker" else mod.stem_layers
        for i in range(nl):
            w.conv_kernel[i] = put(f"ck{i}", params[f"conv{i + 1}"]["kernel"])
            w.conv_bias[i] = put(f"cb{i}", params[f"conv{i + 1}"]["bias"])
            w.norm_scale[i] = put(f"ns{i}", params[f"norm{i + 1}"]["scale"])
            w.norm_bias[i] = put(f"nb{i}", params[f"norm{i + 1}"]["bias"])
        w.norm_pre_scale = put("nps", params["norm_pre"]["scale"])
        w.norm_pre_bias = put("npb", params["norm_pre"]["bias"])
        w.norm_post_scale = put("nqs", params["norm_post"]["scale"])
        w.norm_post_bias = put("nqb", params["norm_post"]["bias"])
        w.head_kernel = put("hk", params["head"]["kernel"])
        w.head_bias = put("hb", params["head"]["bias"])
        self.w = w
        self.buf = _Buffers(device)

    def desc(self, x_shape) -> SimpleDesc:
        m = self.mod
        image = len(x_shape) == 4
        B = x_shape[0]
        T = m.seq_len if image else x_shape[1]
        Hin, Win, Cin = x_shape[-3:]
        return SimpleDesc(B, T, Hin, Win, Cin, int(image), 1 if m.stem_mode == "pathtracker" else 0,
                          m.stem_layers, m.embed_dim,
                          {"gated": 0, "gdn": 1, "no_gate": 2, "add_kqv_1": 3, "deltanet": 4}[m.cssm_type],
                          1 if m.pool_type == "max" else 0, 1 if m.readout_norm == "post" else 0,
                          m.num_classes)

    def block_desc(self, d: SimpleDesc):
        H, W = self.mod.feature_hw(d.Hin, d.Win)
        return self.block.desc((d.B, d.T, H, W, d.embed_dim))

    def stem(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Stem features: (B,H,W,E) for image input, (B,T,H,W,E) for clips.  `out`, when given,
        is a contiguous fp32 tensor of that shape on the same device and receives the result."""
        _require_cuda(x)
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        H, W = self.mod.feature_hw(d.Hin, d.Win)
        shape = (d.B, H, W, d.embed_dim) if d.image_input else (d.B, d.T, H, W, d.embed_dim)
        if out is None:
            feat = torch.empty(shape, dtype=torch.float32, device=x.device)
        else:
            if tuple(out.shape) != shape or out.dtype != torch.float32 or not out.is_contiguous() \
                    or out.device != x.device:
                raise ValueError(f"out must be a contiguous float32 {shape} tensor on {x.device}")
            feat = out
        frames = d.B if d.image_input else d.B * d.T
        half = frames * ((d.Hin + 1) // 2) * ((d.Win + 1) // 2) * d.embed_dim * 4
        ws = self.buf.get("stem", 2 * ((half + 255) // 256 * 256))
        check(self.L.cssm_simple_stem(C.byref(d), C.byref(self.w), x.data_ptr(), feat.data_ptr(),
                                      ws.data_ptr(), ws.numel(), _stream_ptr(self.device)),
              "cssm_simple_stem")
        return feat

    def __call__(self, x: torch.Tensor, last_frame_only: bool = False) -> torch.Tensor:
        """logits (B, num_classes).  last_frame_only=True evaluates the block through its
        last-frame-only entry point (same logits, less work)."""
        _require_cuda(x)
        x = x.contiguous()
        d = self.desc(tuple(x.shape))
        bd = self.block_desc(d)
        pl = self.block.plan(bd)
        n = self.L.cssm_simple_workspace_bytes(C.byref(d), C.byref(bd))
        if n == 0:
            raise NotImplementedError("SimpleCSSM: unsupported shape / field combination")
        ws = self.buf.get("ws", n)
        logits = torch.empty((d.B, d.num_classes), dtype=torch.float32, device=x.device)
        check(self.L.cssm_simple_forward(C.byref(d), C.byref(self.w), C.byref(bd), C.byref(self.block.w),
                                         pl.data_ptr(), x.data_ptr(), logits.data_ptr(),
                                         ws.data_ptr(), n,
                                         SIMPLE_LAST_FRAME_ONLY if last_frame_only else 0,
                                         _stream_ptr(self.device)), "cssm_simple_forward")
        return logits

    def forward_host(self, x_host: torch.Tensor, logits_host: Optional[torch.Tensor] = None,
                     last_frame_only: bool = False) -> torch.Tensor:
        """Host tensors in and out (pinned for full copy speed); returns after the logits have
        arrived in logits_host."""
        if x_host.is_cuda or x_host.dtype != torch.float32:
            raise TypeError("x_host must be a float32 host tensor")
        x_host = x_host.contiguous()
        d = self.desc(tuple(x_host.shape))
        bd = self.block_desc(d)
        pl = self.block.plan(bd)
        n = self.L.cssm_simple_host_workspace_bytes(C.byref(d), C.byref(bd))
        if n == 0:
            raise NotImplementedError("SimpleCSSM: unsupported shape / field combination")
        ws = self.buf.get("hws", n)
        if logits_host is None:
            logits_host = torch.empty((d.B, d.num_classes), dtype=torch.float32)
        check(self.L.cssm_simple_forward_host(C.byref(d), C.byref(self.w), C.byref(bd),
                                              C.byref(self.block.w), pl.data_ptr(),
                                              x_host.data_ptr(), logits_host.data_ptr(),
                                              ws.data_ptr(), n,
                                              SIMPLE_LAST_FRAME_ONLY if last_frame_only else 0,
                                              _stream_ptr(self.device)), "cssm_simple_forward_host")
        _lib.raise_on_device_error("cssm_simple_forward_host")
        return logits_host

    def forward_host_pipelined(self, x_host: torch.Tensor, x_next_host: Optional[torch.Tensor],
                               logits_host: torch.Tensor, last_frame_only: bool = False) -> torch.Tensor:
        """Streaming form of forward_host for a loop over batches: computes the logits of x_host and,
        meanwhile, copies x_next_host (the batch the next call will be given; may be None) to the
        device.  x_next_host must stay unchanged until that next call.  Returns after the logits of
        x_host have arrived."""
        for t in (x_host, x_next_host):
            if t is not None and (t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous()):
                raise TypeError("host batches must be contiguous float32 host tensors")
        if x_next_host is not None and tuple(x_next_host.shape) != tuple(x_host.shape):
            raise ValueError("x_next_host must have the shape of x_host")
        d = self.desc(tuple(x_host.shape))
        bd = self.block_desc(d)
        pl = self.block.plan(bd)
        n = self.L.cssm_simple_host_pipe_workspace_bytes(C.byref(d), C.byref(bd))
        if n == 0:
            raise NotImplementedError("SimpleCSSM: unsupported shape / field combination")
        ws = self.buf.get("pws", n)
        if getattr(self, "_pipe", None) is None:
            h = C.c_void_p()
            check(self.L.cssm_host_pipe_create(C.byref(h)), "cssm_host_pipe_create")
            self._pipe = h
        check(self.L.cssm_simple_forward_host_pipelined(
            C.byref(d), C.byref(self.w), C.byref(bd), C.byref(self.block.w), pl.data_ptr(), self._pipe,
            x_host.data_ptr(), x_next_host.data_ptr() if x_next_host is not None else None,
            logits_host.data_ptr(), ws.data_ptr(), n, SIMPLE_LAST_FRAME_ONLY if last_frame_only else 0,
            _stream_ptr(self.device)), "cssm_simple_forward_host_pipelined")
        _lib.raise_on_device_error("cssm_simple_forward_host_pipelined")
        return logits_host

    def close(self):
        """Waits for a prefetch still in flight and frees the pipe of forward_host_pipelined."""
        if getattr(self, "_pipe", None) is not None:
            self.L.cssm_host_pipe_destroy(self._pipe)
            self._pipe = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
