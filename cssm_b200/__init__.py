"""cssm_b200 — B200 (sm_100a) forward pass of CSSM's gated and GDN spectral token mixers.

The arithmetic lives in libcssm_b200.so (CUDA, C ABI declared in include/cssm_b200.h).
This package holds the ctypes binding and host-side mirrors of the reference's Flax
modules.  Importing the package does not load the library; the first compute call does and
raises if it has not been built."""
from ._lib import CssmError, device_error, lib  # noqa: F401
from .modules import AdditiveCSSM, DeltaNetCSSM, GatedCSSM, GatedDeltaNetCSSM, NoGateCSSM  # noqa: F401
from .simple import SimpleCSSM  # noqa: F401
from .shvit import CSSMSHViT, CSSMSHViTBlock, ConvBlock, cssm_shvit_s1  # noqa: F401

__all__ = ["GatedCSSM", "GatedDeltaNetCSSM", "NoGateCSSM", "AdditiveCSSM", "DeltaNetCSSM", "SimpleCSSM", "CSSMSHViT",
           "CSSMSHViTBlock", "ConvBlock", "cssm_shvit_s1", "CssmError", "device_error", "lib"]
