"""Host-side mirrors of the reference's CSSM-SHViT classifier and of its two block kinds
(src/models/cssm_shvit.py:19-266 `CSSMSHViTBlock`, :269-460 `CSSMSHViT`, :465-474
`cssm_shvit_s1`; src/models/shvit.py:219-262 `ConvBlock`), for the bfloat16 inference forward with
gated mixers.  Field names, defaults, the `apply(variables, x, training=False)` call and the
parameter / batch_stats trees are the reference's; the arithmetic runs in libcssm_b200.so."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import (GATE_ACTS, GATE_TYPES, ROPE_MODES, SHVIT_KINDS, SHVIT_MAX_BLOCKS, ShvitBlockDesc,
                   ShvitBlockWeights, ShvitDesc, ShvitTrace, ShvitWeights, check)
from .modules import _Buffers, _dev_f32, _stream_ptr


def _check_dtype(dtype):
    if str(dtype).replace("torch.", "") not in ("bfloat16", "jnp.bfloat16", "<class 'ml_dtypes.bfloat16'>"):
        raise NotImplementedError(f"CSSM-SHViT: only dtype=bfloat16 has a CUDA path, got {dtype!r} "
                                  "(float32 models: use the block mirrors in cssm_b200.modules)")


def _to_bf16_cuda(x, device):
    if not isinstance(x, torch.Tensor):
        x = torch.from_numpy(np.asarray(x))
    if not x.is_cuda:
        raise TypeError("x must be a CUDA tensor (forward_host takes host arrays); cssm_b200 has no CPU path")
    return x.to(dtype=torch.bfloat16).contiguous()


class _Holder:
    """Keeps the device copies of a parameter tree alive and hands out their addresses."""

    def __init__(self, device):
        self.device = device
        self.t = []

    def __call__(self, arr):
        t = _dev_f32(arr, self.device)
        self.t.append(t)
        return t.data_ptr()


def _fill_gated(w, p, put, gate_type, short_conv_size, short_conv_spatial_size):
    """cssm_gated_weights from the GatedCSSM subtree (src/models/cssm.py:481-584)."""
    w.in_proj_kernel, w.in_proj_bias = put(p["in_proj"]["kernel"]), put(p["in_proj"]["bias"])
    if short_conv_spatial_size > 0:
        w.conv_sp_kernel = put(p["short_conv_spatial"]["kernel"])
        w.conv_sp_bias = put(p["short_conv_spatial"]["bias"])
    if short_conv_size > 0:
        w.conv_t_kernel = put(p["short_conv_temporal"]["kernel"])
        w.conv_t_bias = put(p["short_conv_temporal"]["bias"])
    w.kernel = put(p["kernel"])
    for g, n in enumerate(("delta_proj", "B_proj", "C_proj")):
        if gate_type == "factored":
            w.gate_kernel[2 * g], w.gate_bias[2 * g] = put(p[f"{n}_h"]["kernel"]), put(p[f"{n}_h"]["bias"])
            w.gate_kernel[2 * g + 1], w.gate_bias[2 * g + 1] = put(p[f"{n}_w"]["kernel"]), put(p[f"{n}_w"]["bias"])
        else:
            w.gate_kernel[g], w.gate_bias[g] = put(p[n]["kernel"]), put(p[n]["bias"])
    w.out_proj_kernel, w.out_proj_bias = put(p["out_proj"]["kernel"]), put(p["out_proj"]["bias"])


def _fill_block(w: ShvitBlockWeights, p, put, *, is_cssm, use_pos_conv, use_dwconv, gate_type,
                short_conv_size, short_conv_spatial_size):
    w.norm1_scale, w.norm1_bias = put(p["norm1"]["scale"]), put(p["norm1"]["bias"])
    w.norm2_scale, w.norm2_bias = put(p["norm2"]["scale"]), put(p["norm2"]["bias"])
    w.fc1_kernel, w.fc1_bias = put(p["mlp"]["fc1"]["kernel"]), put(p["mlp"]["fc1"]["bias"])
    w.fc2_kernel, w.fc2_bias = put(p["mlp"]["fc2"]["kernel"]), put(p["mlp"]["fc2"]["bias"])
    if not is_cssm:
        w.dw_kernel, w.dw_bias = put(p["dwconv"]["dwconv"]["kernel"]), put(p["dwconv"]["dwconv"]["bias"])
        w.pw_kernel, w.pw_bias = put(p["pwconv"]["kernel"]), put(p["pwconv"]["bias"])
        return
    if use_pos_conv:
        w.dw_kernel, w.dw_bias = put(p["pos_conv"]["kernel"]), put(p["pos_conv"]["bias"])
    if use_dwconv:
        w.mlp_dw_kernel = put(p["mlp"]["dwconv"]["dwconv"]["kernel"])
        w.mlp_dw_bias = put(p["mlp"]["dwconv"]["dwconv"]["bias"])
    _fill_gated(w.cssm, p["cssm"], put, gate_type, short_conv_size, short_conv_spatial_size)


# ============================================================================ block
@dataclass
class CSSMSHViTBlock:
    """src/models/cssm_shvit.py:19-266 for a 4-D (image) input with cssm_type 'gated'."""
    dim: int
    mlp_ratio: float = 4.0
    drop_path: float = 0.0
    cssm_type: str = "gated"
    dense_mixing: bool = False
    block_size: int = 32
    mixing_rank: int = 0
    gate_activation: str = "softplus"
    num_timesteps: int = 8
    kernel_size: int = 15
    spectral_rho: float = 0.999
    rope_mode: str = "none"
    use_dwconv: bool = True
    output_act: str = "none"
    short_conv_size: int = 4
    short_conv_spatial_size: int = 3
    delta_key_dim: int = 2
    output_norm: str = "rms"
    gate_type: str = "factored"
    block_norm: str = "global_layer"
    use_pos_conv: bool = True
    gate_proj_bias_init: float = 0.0
    static_image_fast_path: bool = False
    use_input_gates: bool = True
    ssl_proj_dim: int = 0
    timestep_gate: bool = False
    dtype: Any = "bfloat16"
    param_dtype: Any = "float32"
    is_cssm: bool = True
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    def _check_fields(self):
        bad = []
        if self.cssm_type != "gated":
            bad.append(f"cssm_type={self.cssm_type!r}")
        if self.dense_mixing or self.mixing_rank:
            bad.append("dense_mixing / mixing_rank")
        if self.block_norm != "global_layer":
            bad.append(f"block_norm={self.block_norm!r}")
        if self.output_act != "none":
            bad.append(f"output_act={self.output_act!r}")
        if self.timestep_gate or self.ssl_proj_dim:
            bad.append("timestep_gate / ssl_proj_dim")
        if self.gate_type not in GATE_TYPES or self.rope_mode not in ROPE_MODES:
            bad.append("gate_type / rope_mode")
        if bad:
            raise NotImplementedError("CSSMSHViTBlock: no CUDA kernel for " + "; ".join(bad))
        _check_dtype(self.dtype)

    def desc(self, shape) -> ShvitBlockDesc:
        B, H, W, Cc = shape
        if Cc != self.dim:
            raise ValueError(f"x has {Cc} channels, block has {self.dim}")
        return ShvitBlockDesc(B, H, W, Cc, 1 if self.is_cssm else 0, int(self.dim * self.mlp_ratio),
                              self.num_timesteps, self.kernel_size, int(self.use_pos_conv),
                              int(self.use_dwconv), ROPE_MODES[self.rope_mode], 10000.0,
                              float(self.spectral_rho), GATE_ACTS.get(self.gate_activation, 0),
                              self.short_conv_size, self.short_conv_spatial_size,
                              GATE_TYPES[self.gate_type])

    def bind(self, variables, device="cuda") -> "BoundBlock":
        self._check_fields()
        return BoundBlock(self, variables["params"] if "params" in variables else variables,
                          torch.device(device))

    def apply(self, variables, x, deterministic: bool = True):
        """y = block.apply({'params': tree}, x): x (B,H,W,C) CUDA tensor, returns bfloat16."""
        if not deterministic:
            raise NotImplementedError("inference only")
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


@dataclass
class ConvBlock(CSSMSHViTBlock):
    """src/models/shvit.py:219-262: LayerNorm -> depthwise 7x7 -> gelu -> Dense + residual, then
    LayerNorm -> Mlp (no depthwise conv) + residual."""
    is_cssm: bool = False

    def _check_fields(self):
        _check_dtype(self.dtype)


class BoundBlock:
    def __init__(self, mod: CSSMSHViTBlock, p, device):
        self.mod, self.device, self.variables_ref = mod, device, None
        self.L = _lib.lib()
        self.hold = _Holder(device)
        self.w = ShvitBlockWeights()
        _fill_block(self.w, p, self.hold, is_cssm=mod.is_cssm, use_pos_conv=mod.use_pos_conv,
                    use_dwconv=mod.use_dwconv, gate_type=mod.gate_type,
                    short_conv_size=mod.short_conv_size,
                    short_conv_spatial_size=mod.short_conv_spatial_size)
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}

    def plan(self, d):
        key = (d.B, d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_shvit_block_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError(f"{type(self.mod).__name__}: no CUDA kernel for these fields / shape")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_shvit_block_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                                    _stream_ptr(self.device)), "cssm_shvit_block_plan_init")
            self._plans[key] = pl
        return pl

    def __call__(self, x):
        x = _to_bf16_cuda(x, self.device)
        d = self.mod.desc(tuple(x.shape))
        pl = self.plan(d)
        n = self.L.cssm_shvit_block_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws", n)
        y = torch.empty_like(x)
        check(self.L.cssm_shvit_block_forward(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                              y.data_ptr(), ws.data_ptr(), n, _stream_ptr(self.device)),
              "cssm_shvit_block_forward")
        return y


# ============================================================================ model
@dataclass
class CSSMSHViT:
    """src/models/cssm_shvit.py:269-460 (field names and defaults), image input, gated mixers."""
    num_classes: int = 1000
    embed_dims: Sequence[int] = (128, 256, 384, 512)
    depths: Sequence[int] = (1, 2, 4, 1)
    mlp_ratio: float = 4.0
    drop_rate: float = 0.0
    drop_path_rate: float = 0.1
    use_cssm_stages: Sequence[bool] = (False, False, True, True)
    cssm_type: str = "gated"
    dense_mixing: bool = False
    block_size: int = 32
    mixing_rank: int = 0
    gate_activation: str = "softplus"
    num_timesteps: int = 8
    kernel_sizes: Sequence[int] = (15, 15, 5, 3)
    spectral_rho: float = 0.999
    rope_mode: str = "none"
    use_dwconv: bool = True
    output_act: str = "none"
    short_conv_size: int = 4
    short_conv_spatial_size: int = 3
    delta_key_dim: int = 2
    output_norm: str = "rms"
    gate_type: str = "factored"
    block_norm: str = "global_layer"
    use_pos_conv: bool = True
    gate_proj_bias_init: float = 0.0
    head_pool: str = "max"
    static_image_fast_path: bool = False
    use_input_gates: bool = True
    ssl_proj_dim: int = 0
    linear_probe: bool = False
    timestep_gate: bool = False
    dtype: Any = "bfloat16"
    param_dtype: Any = "float32"
    _bound: Dict[Any, Any] = field(default_factory=dict, repr=False, compare=False)

    def _check_fields(self):
        bad = []
        if self.cssm_type != "gated":
            bad.append(f"cssm_type={self.cssm_type!r}")
        if self.dense_mixing or self.mixing_rank:
            bad.append("dense_mixing / mixing_rank")
        if self.block_norm != "global_layer" or self.output_act != "none":
            bad.append("block_norm / output_act")
        if self.timestep_gate or self.ssl_proj_dim or self.linear_probe:
            bad.append("timestep_gate / ssl_proj_dim / linear_probe")
        if self.head_pool not in ("max", "mean"):
            bad.append(f"head_pool={self.head_pool!r}")
        if sum(self.depths) > SHVIT_MAX_BLOCKS:
            bad.append(f"more than {SHVIT_MAX_BLOCKS} blocks")
        if bad:
            raise NotImplementedError("CSSMSHViT: no CUDA kernel for " + "; ".join(bad))
        _check_dtype(self.dtype)

    def desc(self, shape) -> ShvitDesc:
        B, H, W, Cin = shape
        i4 = C.c_int32 * 4
        return ShvitDesc(B, H, W, Cin, i4(*self.embed_dims), i4(*self.depths),
                         i4(*[int(u) for u in self.use_cssm_stages]), i4(*self.kernel_sizes),
                         self.num_classes, self.num_timesteps, float(self.mlp_ratio),
                         int(self.use_pos_conv), int(self.use_dwconv), 0 if self.head_pool == "max" else 1,
                         ROPE_MODES[self.rope_mode], 10000.0, float(self.spectral_rho),
                         GATE_ACTS.get(self.gate_activation, 0), self.short_conv_size,
                         self.short_conv_spatial_size, GATE_TYPES[self.gate_type])

    def bind(self, variables, device="cuda") -> "BoundShvit":
        self._check_fields()
        return BoundShvit(self, variables["params"], variables["batch_stats"], torch.device(device))

    def apply(self, variables, x, training: bool = False):
        """logits = model.apply({'params': ..., 'batch_stats': ...}, x, training=False)."""
        if training:
            raise NotImplementedError("CSSMSHViT: inference only")
        key = id(variables)
        bound = self._bound.get(key)
        if bound is None or bound.variables_ref is not variables:
            bound = self.bind(variables, x.device)
            bound.variables_ref = variables
            self._bound.clear()
            self._bound[key] = bound
        return bound(x)


def cssm_shvit_s1(num_classes: int = 1000, num_timesteps: int = 8, cssm_type: str = "gated", **kwargs):
    """src/models/cssm_shvit.py:465-474."""
    return CSSMSHViT(num_classes=num_classes, embed_dims=(64, 128, 256, 384), depths=(1, 2, 2, 1),
                     num_timesteps=num_timesteps, cssm_type=cssm_type, **kwargs)


class BoundShvit:
    def __init__(self, mod: CSSMSHViT, p, s, device):
        self.mod, self.device, self.variables_ref = mod, device, None
        self.L = _lib.lib()
        self.hold = put = _Holder(device)
        w = ShvitWeights()

        def convbn(dst, pp, ss):
            dst.kernel = put(pp["conv"]["kernel"])
            dst.bn_scale, dst.bn_bias = put(pp["bn"]["scale"]), put(pp["bn"]["bias"])
            dst.bn_mean, dst.bn_var = put(ss["bn"]["mean"]), put(ss["bn"]["var"])

        convbn(w.patch[0], p["patch_embed"]["ConvBN_0"], s["patch_embed"]["ConvBN_0"])
        convbn(w.patch[1], p["patch_embed"]["ConvBN_1"], s["patch_embed"]["ConvBN_1"])
        for i in (1, 2, 3):
            convbn(w.down[i - 1], p[f"downsample{i}"]["ConvBN_0"], s[f"downsample{i}"]["ConvBN_0"])
        bi = 0
        for st in range(4):
            for b in range(mod.depths[st]):
                _fill_block(w.blocks[bi], p[f"stage{st}_block{b}"], put,
                            is_cssm=bool(mod.use_cssm_stages[st]), use_pos_conv=mod.use_pos_conv,
                            use_dwconv=mod.use_dwconv, gate_type=mod.gate_type,
                            short_conv_size=mod.short_conv_size,
                            short_conv_spatial_size=mod.short_conv_spatial_size)
                bi += 1
        w.norm_scale, w.norm_bias = put(p["norm"]["scale"]), put(p["norm"]["bias"])
        w.head_kernel, w.head_bias = put(p["head"]["kernel"]), put(p["head"]["bias"])
        self.w = w
        self.buf = _Buffers(device)
        self._plans: Dict[Any, torch.Tensor] = {}
        self._pipe = None

    def desc(self, shape):
        return self.mod.desc(shape)

    def plan(self, d):
        key = (d.B, d.H, d.W)
        pl = self._plans.get(key)
        if pl is None:
            n = self.L.cssm_shvit_plan_bytes(C.byref(d))
            if n == 0:
                raise NotImplementedError("CSSMSHViT: no CUDA kernel for these fields / shape")
            pl = torch.empty(n, dtype=torch.uint8, device=self.device)
            check(self.L.cssm_shvit_plan_init(C.byref(d), C.byref(self.w), pl.data_ptr(), n,
                                              _stream_ptr(self.device)), "cssm_shvit_plan_init")
            self._plans[key] = pl
        return pl

    def workspace(self, d, host=False):
        fn = self.L.cssm_shvit_host_workspace_bytes if host else self.L.cssm_shvit_workspace_bytes
        n = fn(C.byref(d))
        return self.buf.get("ws_host" if host else "ws", n), n

    def __call__(self, x, out=None):
        x = _to_bf16_cuda(x, self.device)
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        ws, n = self.workspace(d)
        logits = torch.empty((d.B, d.num_classes), dtype=torch.float32, device=self.device) if out is None else out
        check(self.L.cssm_shvit_forward(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                        logits.data_ptr(), ws.data_ptr(), n, _stream_ptr(self.device)),
              "cssm_shvit_forward")
        return logits

    def forward_traced(self, x, out=None, capacity: int = 256):
        """One forward with an event before every kernel launch.  Returns (logits, launches) where
        launches is a list of (kernel kind, milliseconds, algorithmic bytes) in launch order."""
        x = _to_bf16_cuda(x, self.device)
        d = self.desc(tuple(x.shape))
        pl = self.plan(d)
        ws, n = self.workspace(d)
        logits = torch.empty((d.B, d.num_classes), dtype=torch.float32, device=self.device) if out is None else out
        stream = torch.cuda.current_stream(self.device)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(capacity)]
        for e in evs:
            e.record(stream)                      # creates the raw cudaEvent_t handles
        torch.cuda.synchronize(self.device)
        tr = ShvitTrace((C.c_void_p * capacity)(*[e.cuda_event for e in evs]),
                        (C.c_int32 * capacity)(), (C.c_double * capacity)(), capacity, 0)
        check(self.L.cssm_shvit_forward_timed(C.byref(d), C.byref(self.w), pl.data_ptr(), x.data_ptr(),
                                              logits.data_ptr(), ws.data_ptr(), n, stream.cuda_stream,
                                              C.byref(tr)), "cssm_shvit_forward_timed")
        torch.cuda.synchronize(self.device)
        launches = [(SHVIT_KINDS[tr.kinds[i]], evs[i].elapsed_time(evs[i + 1]), tr.bytes[i])
                    for i in range(tr.count - 1)]
        return logits, launches

    def forward_host(self, x_host: torch.Tensor, logits_host: torch.Tensor):
        """x_host: (B,H,W,Cin) bfloat16 host tensor (pinned for full copy speed); logits_host:
        (B,num_classes) float32 host tensor.  Returns after the logits have arrived."""
        d = self.desc(tuple(x_host.shape))
        pl = self.plan(d)
        ws, n = self.workspace(d, host=True)
        check(self.L.cssm_shvit_forward_host(C.byref(d), C.byref(self.w), pl.data_ptr(), x_host.data_ptr(),
                                             logits_host.data_ptr(), ws.data_ptr(), n,
                                             _stream_ptr(self.device)), "cssm_shvit_forward_host")
        _lib.raise_on_device_error("cssm_shvit_forward_host")
        return logits_host

    def forward_host_pipelined(self, x_host: torch.Tensor, x_next_host: Optional[torch.Tensor],
                               logits_host: torch.Tensor):
        """Streaming form of forward_host for a loop over batches: computes the logits of x_host and,
        meanwhile, copies x_next_host (the batch the next call will be given; may be None) to the
        device.  x_next_host must stay unchanged until that next call.  Returns after the logits of
        x_host have arrived."""
        d = self.desc(tuple(x_host.shape))
        if x_next_host is not None and tuple(x_next_host.shape) != tuple(x_host.shape):
            raise ValueError("x_next_host must have the shape of x_host")
        pl = self.plan(d)
        n = self.L.cssm_shvit_host_pipe_workspace_bytes(C.byref(d))
        ws = self.buf.get("ws_pipe", n)
        if self._pipe is None:
            h = C.c_void_p()
            check(self.L.cssm_host_pipe_create(C.byref(h)), "cssm_host_pipe_create")
            self._pipe = h
        check(self.L.cssm_shvit_forward_host_pipelined(
            C.byref(d), C.byref(self.w), pl.data_ptr(), self._pipe, x_host.data_ptr(),
            x_next_host.data_ptr() if x_next_host is not None else None, logits_host.data_ptr(),
            ws.data_ptr(), n, _stream_ptr(self.device)), "cssm_shvit_forward_host_pipelined")
        _lib.raise_on_device_error("cssm_shvit_forward_host_pipelined")
        return logits_host

    def close(self):
        """Waits for a prefetch still in flight and frees the pipe of forward_host_pipelined."""
        if self._pipe is not None:
            self.L.cssm_host_pipe_destroy(self._pipe)
            self._pipe = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
