"""`jax.numpy` stand-in: NumPy itself, with the dtype aliases the wide mode needs."""
from __future__ import annotations

import numpy as _np
from numpy import *  # noqa: F401,F403
from numpy import fft, linalg  # noqa: F401

try:
    import ml_dtypes as _ml
    bfloat16 = _ml.bfloat16
    float8_e4m3fn = _ml.float8_e4m3fn
    float8_e5m2 = _ml.float8_e5m2
except ImportError:  # pragma: no cover
    bfloat16 = float8_e4m3fn = float8_e5m2 = None

ndarray = _np.ndarray
newaxis = None
pi = _np.pi
inf = _np.inf
int32 = _np.int32
float16 = _np.float16
float64 = _np.float64
complex128 = _np.complex128
import os as _os

_WIDE = _os.environ.get("CSSM_SHIM_WIDE", "1") != "0"
float32 = _np.float64 if _WIDE else _np.float32
complex64 = _np.complex128 if _WIDE else _np.complex64


def _set_wide(wide: bool):
    global float32, complex64
    float32 = _np.float64 if wide else _np.float32
    complex64 = _np.complex128 if wide else _np.complex64


def dtype(x):
    return _np.dtype(x)


def asarray(x, dtype=None):
    return _np.asarray(x, dtype=dtype)


def array(x, dtype=None):
    return _np.array(x, dtype=dtype)


def iscomplexobj(x):
    return _np.iscomplexobj(x)


def finfo(dt):
    if bfloat16 is not None and _np.dtype(dt) == _np.dtype(bfloat16):
        return _ml.finfo(dt)
    return _np.finfo(dt)
