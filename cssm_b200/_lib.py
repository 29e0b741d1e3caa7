"""ctypes binding of libcssm_b200.so.  There is no fallback: if the library is missing the
import of anything that computes raises, telling the user to build it."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcssm_b200.so")

ROPE_MODES = {"none": 0, "spatiotemporal": 1, "temporal": 2, "spatial_only": 3, "mrope": 4}
GATE_TYPES = {"dense": 0, "factored": 1}
DELTANET_GATE_TYPES = {"dense": 0, "factored": 1, "channel": 2}
GDN_GATE_TYPES = {"dense": 0, "factored": 1, "channel": 2, "scalar": 3}
GATE_ACTS = {"softplus": 0, "sigmoid": 1, "exp": 2}


class CssmError(RuntimeError):
    pass


class GatedDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("C", C.c_int32), ("kernel_size", C.c_int32), ("rope_mode", C.c_int32),
                ("rope_base", C.c_float), ("spectral_rho", C.c_float),
                ("gate_activation", C.c_int32), ("short_conv_size", C.c_int32),
                ("short_conv_spatial_size", C.c_int32), ("gate_type", C.c_int32)]


class GatedWeights(C.Structure):
    _fields_ = [("in_proj_kernel", C.c_void_p), ("in_proj_bias", C.c_void_p),
                ("conv_sp_kernel", C.c_void_p), ("conv_sp_bias", C.c_void_p),
                ("conv_t_kernel", C.c_void_p), ("conv_t_bias", C.c_void_p),
                ("kernel", C.c_void_p),
                ("gate_kernel", C.c_void_p * 6), ("gate_bias", C.c_void_p * 6),
                ("out_proj_kernel", C.c_void_p), ("out_proj_bias", C.c_void_p)]


class ShvitBlockDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("W", C.c_int32), ("C", C.c_int32),
                ("is_cssm", C.c_int32), ("hidden", C.c_int32), ("num_timesteps", C.c_int32),
                ("kernel_size", C.c_int32), ("use_pos_conv", C.c_int32), ("use_dwconv", C.c_int32),
                ("rope_mode", C.c_int32), ("rope_base", C.c_float), ("spectral_rho", C.c_float),
                ("gate_activation", C.c_int32), ("short_conv_size", C.c_int32),
                ("short_conv_spatial_size", C.c_int32), ("gate_type", C.c_int32)]


class ShvitBlockWeights(C.Structure):
    _fields_ = [("norm1_scale", C.c_void_p), ("norm1_bias", C.c_void_p),
                ("norm2_scale", C.c_void_p), ("norm2_bias", C.c_void_p),
                ("dw_kernel", C.c_void_p), ("dw_bias", C.c_void_p),
                ("pw_kernel", C.c_void_p), ("pw_bias", C.c_void_p),
                ("fc1_kernel", C.c_void_p), ("fc1_bias", C.c_void_p),
                ("fc2_kernel", C.c_void_p), ("fc2_bias", C.c_void_p),
                ("mlp_dw_kernel", C.c_void_p), ("mlp_dw_bias", C.c_void_p),
                ("cssm", GatedWeights)]


class ShvitConvBN(C.Structure):
    _fields_ = [("kernel", C.c_void_p), ("bn_scale", C.c_void_p), ("bn_bias", C.c_void_p),
                ("bn_mean", C.c_void_p), ("bn_var", C.c_void_p)]


SHVIT_MAX_BLOCKS = 16


class ShvitDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("W", C.c_int32), ("Cin", C.c_int32),
                ("embed_dims", C.c_int32 * 4), ("depths", C.c_int32 * 4),
                ("use_cssm", C.c_int32 * 4), ("kernel_sizes", C.c_int32 * 4),
                ("num_classes", C.c_int32), ("num_timesteps", C.c_int32), ("mlp_ratio", C.c_float),
                ("use_pos_conv", C.c_int32), ("use_dwconv", C.c_int32), ("head_pool", C.c_int32),
                ("rope_mode", C.c_int32), ("rope_base", C.c_float), ("spectral_rho", C.c_float),
                ("gate_activation", C.c_int32), ("short_conv_size", C.c_int32),
                ("short_conv_spatial_size", C.c_int32), ("gate_type", C.c_int32)]


class ShvitWeights(C.Structure):
    _fields_ = [("patch", ShvitConvBN * 2), ("down", ShvitConvBN * 3),
                ("blocks", ShvitBlockWeights * SHVIT_MAX_BLOCKS),
                ("norm_scale", C.c_void_p), ("norm_bias", C.c_void_p),
                ("head_kernel", C.c_void_p), ("head_bias", C.c_void_p)]


class ShvitTrace(C.Structure):
    _fields_ = [("events", C.POINTER(C.c_void_p)), ("kinds", C.POINTER(C.c_int32)),
                ("bytes", C.POINTER(C.c_double)), ("capacity", C.c_int32), ("count", C.c_int32)]


SHVIT_KINDS = ["stem_conv", "conv_gemm", "gemm", "layernorm", "dwconv7", "dwconv3", "sample_norm",
               "plane_sum", "gates", "spectral", "pool", "head", "mixer_f32", "add_res", "mlp", "end"]


class GatedWsLayout(C.Structure):
    _fields_ = [("xz_planar", C.c_size_t), ("ctx_sum", C.c_size_t),
                ("gate_maps", C.c_size_t), ("total", C.c_size_t)]


class GdnDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("C", C.c_int32), ("delta_key_dim", C.c_int32), ("kernel_size", C.c_int32),
                ("rope_mode", C.c_int32), ("rope_base", C.c_float), ("spectral_rho", C.c_float),
                ("gate_type", C.c_int32), ("short_conv_size", C.c_int32),
                ("output_norm", C.c_int32), ("use_input_gates", C.c_int32),
                ("output_gate_act", C.c_int32), ("use_spectral_l2_norm", C.c_int32),
                ("qkv_conv_size", C.c_int32), ("no_spectral_clamp", C.c_int32)]


class GdnWeights(C.Structure):
    _fields_ = [("kernel", C.c_void_p),
                ("qkv_dw_kernel", C.c_void_p), ("qkv_dw_bias", C.c_void_p),
                ("qkv_proj_kernel", C.c_void_p), ("qkv_proj_bias", C.c_void_p),
                ("conv_t_kernel", C.c_void_p * 3), ("conv_t_bias", C.c_void_p * 3),
                ("gate_kernel", C.c_void_p * 8), ("gate_bias", C.c_void_p * 8),
                ("gate_proj_kernel", C.c_void_p), ("gate_proj_bias", C.c_void_p),
                ("rms_scale", C.c_void_p),
                ("output_proj_kernel", C.c_void_p), ("output_proj_bias", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/cssm_b200.h declares
_P = C.c_void_p
class NoGateDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("C", C.c_int32), ("kernel_size", C.c_int32), ("spectral_rho", C.c_float)]


class NoGateWeights(C.Structure):
    _fields_ = [("kernel", C.c_void_p), ("out_proj_kernel", C.c_void_p), ("out_proj_bias", C.c_void_p)]


class AdditiveDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("C", C.c_int32), ("kernel_size", C.c_int32), ("rope_mode", C.c_int32),
                ("rope_base", C.c_float), ("spectral_rho", C.c_float), ("gate_type", C.c_int32),
                ("single_state", C.c_int32), ("goom_floor", C.c_int32)]


class AdditiveWeights(C.Structure):
    _fields_ = [("kernel", C.c_void_p), ("x_proj_kernel", C.c_void_p), ("x_proj_bias", C.c_void_p),
                ("gate_kernel", C.c_void_p * 6), ("gate_bias", C.c_void_p * 6),
                ("output_proj_kernel", C.c_void_p), ("output_proj_bias", C.c_void_p)]


class DeltaNetDesc(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("C", C.c_int32), ("kernel_size", C.c_int32), ("rope_mode", C.c_int32),
                ("rope_base", C.c_float), ("spectral_rho", C.c_float), ("gate_type", C.c_int32),
                ("goom_floor", C.c_int32)]


class DeltaNetWeights(C.Structure):
    _fields_ = [("kernel", C.c_void_p), ("qkv_proj_kernel", C.c_void_p), ("qkv_proj_bias", C.c_void_p),
                ("gate_kernel", C.c_void_p * 10), ("gate_bias", C.c_void_p * 10),
                ("output_proj_kernel", C.c_void_p), ("output_proj_bias", C.c_void_p)]


class SimpleDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("B", "T", "Hin", "Win", "Cin", "image_input", "stem_mode", "stem_layers",
                 "embed_dim", "block", "pool_type", "readout_norm", "num_classes")]


class SimpleWeights(C.Structure):
    _fields_ = [("conv_kernel", C.c_void_p * 4), ("conv_bias", C.c_void_p * 4),
                ("norm_scale", C.c_void_p * 4), ("norm_bias", C.c_void_p * 4),
                ("norm_pre_scale", C.c_void_p), ("norm_pre_bias", C.c_void_p),
                ("norm_post_scale", C.c_void_p), ("norm_post_bias", C.c_void_p),
                ("head_kernel", C.c_void_p), ("head_bias", C.c_void_p)]


SIMPLE_LAST_FRAME_ONLY = 1

SIGNATURES = {
    "cssm_strerror": (C.c_char_p, [C.c_int]),
    "cssm_last_cuda_error": (C.c_char_p, []),
    "cssm_version": (C.c_char_p, []),
    "cssm_gated_plan_bytes": (C.c_size_t, [C.POINTER(GatedDesc)]),
    "cssm_gated_workspace_bytes": (C.c_size_t, [C.POINTER(GatedDesc)]),
    "cssm_gated_plan_init": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P,
                                       C.c_size_t, _P]),
    "cssm_gated_forward": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P,
                                     _P, C.c_size_t, _P]),
    "cssm_gated_forward_last": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P,
                                          _P, C.c_size_t, _P]),
    "cssm_gated_bf16_workspace_bytes": (C.c_size_t, [C.POINTER(GatedDesc)]),
    "cssm_gated_forward_bf16": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P,
                                          C.c_int32, _P, C.c_size_t, _P]),
    "cssm_gated_host_workspace_bytes": (C.c_size_t, [C.POINTER(GatedDesc), C.c_int32]),
    "cssm_gated_forward_host": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P,
                                          _P, C.c_int32, _P, C.c_size_t, _P]),
    "cssm_gated_in_proj": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P, _P]),
    "cssm_gated_short_conv": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P]),
    "cssm_gated_gates": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P]),
    "cssm_gated_spectral": (C.c_int, [C.POINTER(GatedDesc), _P, _P, _P, _P]),
    "cssm_gated_out_proj": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P, _P]),
    "cssm_gated_workspace_layout": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWsLayout)]),
    "cssm_gdn_plan_bytes": (C.c_size_t, [C.POINTER(GdnDesc)]),
    "cssm_gdn_workspace_bytes": (C.c_size_t, [C.POINTER(GdnDesc)]),
    "cssm_gdn_plan_init": (C.c_int, [C.POINTER(GdnDesc), C.POINTER(GdnWeights), _P, C.c_size_t, _P]),
    "cssm_gdn_forward": (C.c_int, [C.POINTER(GdnDesc), C.POINTER(GdnWeights), _P, _P, _P, _P,
                                   C.c_size_t, _P]),
    "cssm_gdn_forward_timed": (C.c_int, [C.POINTER(GdnDesc), C.POINTER(GdnWeights), _P, _P, _P, _P,
                                         C.c_size_t, _P, C.POINTER(C.c_void_p)]),
    "cssm_gdn_forward_last": (C.c_int, [C.POINTER(GdnDesc), C.POINTER(GdnWeights), _P, _P, _P, _P,
                                        C.c_size_t, _P]),
    "cssm_gdn_forward_static_image": (C.c_int, [C.POINTER(GdnDesc), C.POINTER(GdnWeights), _P, _P, _P,
                                                _P, C.c_size_t, _P]),
    "cssm_nogate_plan_bytes": (C.c_size_t, [C.POINTER(NoGateDesc)]),
    "cssm_nogate_workspace_bytes": (C.c_size_t, [C.POINTER(NoGateDesc)]),
    "cssm_nogate_plan_init": (C.c_int, [C.POINTER(NoGateDesc), C.POINTER(NoGateWeights), _P, C.c_size_t, _P]),
    "cssm_nogate_forward": (C.c_int, [C.POINTER(NoGateDesc), C.POINTER(NoGateWeights), _P, _P, _P, _P,
                                      C.c_size_t, _P]),
    "cssm_additive_plan_bytes": (C.c_size_t, [C.POINTER(AdditiveDesc)]),
    "cssm_additive_workspace_bytes": (C.c_size_t, [C.POINTER(AdditiveDesc)]),
    "cssm_additive_plan_init": (C.c_int, [C.POINTER(AdditiveDesc), C.POINTER(AdditiveWeights), _P,
                                          C.c_size_t, _P]),
    "cssm_additive_forward": (C.c_int, [C.POINTER(AdditiveDesc), C.POINTER(AdditiveWeights), _P, _P,
                                        _P, _P, C.c_size_t, _P]),
    "cssm_deltanet_plan_bytes": (C.c_size_t, [C.POINTER(DeltaNetDesc)]),
    "cssm_deltanet_workspace_bytes": (C.c_size_t, [C.POINTER(DeltaNetDesc)]),
    "cssm_deltanet_plan_init": (C.c_int, [C.POINTER(DeltaNetDesc), C.POINTER(DeltaNetWeights), _P,
                                          C.c_size_t, _P]),
    "cssm_deltanet_forward": (C.c_int, [C.POINTER(DeltaNetDesc), C.POINTER(DeltaNetWeights), _P, _P,
                                        _P, _P, C.c_size_t, _P]),
    "cssm_simple_workspace_bytes": (C.c_size_t, [C.POINTER(SimpleDesc), _P]),
    "cssm_simple_stem": (C.c_int, [C.POINTER(SimpleDesc), C.POINTER(SimpleWeights), _P, _P, _P,
                                   C.c_size_t, _P]),
    "cssm_simple_readout": (C.c_int, [C.POINTER(SimpleDesc), C.POINTER(SimpleWeights), C.c_int32,
                                      C.c_int32, _P, C.c_size_t, _P, C.c_size_t, _P, _P, _P]),
    "cssm_simple_forward": (C.c_int, [C.POINTER(SimpleDesc), C.POINTER(SimpleWeights), _P, _P, _P,
                                      _P, _P, _P, C.c_size_t, C.c_int32, _P]),
    "cssm_simple_host_workspace_bytes": (C.c_size_t, [C.POINTER(SimpleDesc), _P]),
    "cssm_simple_forward_host": (C.c_int, [C.POINTER(SimpleDesc), C.POINTER(SimpleWeights), _P, _P,
                                           _P, _P, _P, _P, C.c_size_t, C.c_int32, _P]),
    "cssm_simple_host_pipe_workspace_bytes": (C.c_size_t, [C.POINTER(SimpleDesc), _P]),
    "cssm_simple_forward_host_pipelined": (C.c_int, [C.POINTER(SimpleDesc), C.POINTER(SimpleWeights), _P, _P,
                                                     _P, _P, _P, _P, _P, _P, C.c_size_t, C.c_int32, _P]),
    "cssm_device_error": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "cssm_shvit_block_plan_bytes": (C.c_size_t, [C.POINTER(ShvitBlockDesc)]),
    "cssm_shvit_block_workspace_bytes": (C.c_size_t, [C.POINTER(ShvitBlockDesc)]),
    "cssm_shvit_block_plan_init": (C.c_int, [C.POINTER(ShvitBlockDesc), C.POINTER(ShvitBlockWeights), _P,
                                             C.c_size_t, _P]),
    "cssm_shvit_block_forward": (C.c_int, [C.POINTER(ShvitBlockDesc), C.POINTER(ShvitBlockWeights), _P,
                                           _P, _P, _P, C.c_size_t, _P]),
    "cssm_shvit_plan_bytes": (C.c_size_t, [C.POINTER(ShvitDesc)]),
    "cssm_shvit_workspace_bytes": (C.c_size_t, [C.POINTER(ShvitDesc)]),
    "cssm_shvit_plan_init": (C.c_int, [C.POINTER(ShvitDesc), C.POINTER(ShvitWeights), _P, C.c_size_t, _P]),
    "cssm_shvit_forward": (C.c_int, [C.POINTER(ShvitDesc), C.POINTER(ShvitWeights), _P, _P, _P, _P,
                                     C.c_size_t, _P]),
    "cssm_shvit_forward_timed": (C.c_int, [C.POINTER(ShvitDesc), C.POINTER(ShvitWeights), _P, _P, _P, _P,
                                           C.c_size_t, _P, C.POINTER(ShvitTrace)]),
    "cssm_shvit_host_workspace_bytes": (C.c_size_t, [C.POINTER(ShvitDesc)]),
    "cssm_shvit_forward_host": (C.c_int, [C.POINTER(ShvitDesc), C.POINTER(ShvitWeights), _P, _P, _P, _P,
                                          C.c_size_t, _P]),
    "cssm_host_pipe_create": (C.c_int, [C.POINTER(_P)]),
    "cssm_host_pipe_destroy": (C.c_int, [_P]),
    "cssm_shvit_host_pipe_workspace_bytes": (C.c_size_t, [C.POINTER(ShvitDesc)]),
    "cssm_shvit_forward_host_pipelined": (C.c_int, [C.POINTER(ShvitDesc), C.POINTER(ShvitWeights), _P, _P, _P, _P,
                                                    _P, _P, C.c_size_t, _P]),
    "cssm_bf16_packed_ld": (C.c_int32, [C.c_int32]),
    "cssm_bf16_pack_weight": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, _P]),
    "cssm_bf16_gemm": (C.c_int, [_P, C.c_int32, C.c_int32, _P, C.c_int32, _P, C.c_int32, _P, _P, _P]),
    "cssm_bf16_mlp": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P, _P]),
    "cssm_bf16_conv3x3s2_packed_ld": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32]),
    "cssm_bf16_pack_conv3x3s2_weight": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P]),
    "cssm_bf16_conv3x3s2": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, C.c_int32, _P,
                                      C.c_int32, _P, _P]),
    "cssm_static_scratch_bytes": (C.c_size_t, []),
    "cssm_gated_forward_static": (C.c_int, [C.POINTER(GatedDesc), C.POINTER(GatedWeights), _P, _P,
                                            _P, _P]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises CssmError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CssmError(
                f"{LIB_PATH} is missing: build it with `python -m cssm_b200.build` "
                "(needs nvcc).  cssm_b200 has no CPU or PyTorch fallback.")
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)          # AttributeError here = header/library mismatch
            fn.restype = res
            fn.argtypes = args
        _lib = h
    return _lib


def device_error(clear: bool = True) -> int:
    """The device error word: non-zero when a bounded wait inside a kernel expired since the last
    clearing read (bits 0-7 fp32 GEMM, 8-15 fused spectral kernel, 16-23 bf16 GEMM, 24-31 fused MLP).  Reading it
    waits for the device, so the mirrors call it only where they wait anyway (host entry points)."""
    L = lib()
    word = C.c_int(0)
    check(L.cssm_device_error(C.byref(word), 1 if clear else 0), "cssm_device_error")
    return int(word.value)


def raise_on_device_error(what: str) -> None:
    word = device_error(clear=True)
    if word:
        raise CssmError(f"{what}: a bounded device-side wait expired (error word 0x{word:x}); "
                        "the results of the call are not valid")


def check(status: int, what: str) -> None:
    if status != 0:
        L = lib()
        msg = L.cssm_strerror(status).decode()
        extra = L.cssm_last_cuda_error().decode() if status == 6 else ""
        raise CssmError(f"{what}: {msg} (status {status}) {extra}".strip())
