"""`flax.linen.initializers` stand-ins (NumPy generator behind the key; see jax/random.py)."""
from __future__ import annotations

import numpy as np

from jax import random as _jr


def _dt(dtype):
    import jax.numpy as jnp
    return dtype or jnp.float32


def zeros(key, shape, dtype=None):
    return np.zeros(shape, _dt(dtype))


def ones(key, shape, dtype=None):
    return np.ones(shape, _dt(dtype))


def zeros_init():
    return zeros


def ones_init():
    return ones


def constant(value):
    return lambda key, shape, dtype=None: np.full(shape, value, _dt(dtype))


def normal(stddev=1e-2):
    return lambda key, shape, dtype=None: (_jr.normal(key, shape) * stddev).astype(_dt(dtype))


def uniform(scale=1e-2):
    return lambda key, shape, dtype=None: (_jr.uniform(key, shape) * scale).astype(_dt(dtype))


def _fans(shape):
    if len(shape) < 1:
        return 1.0, 1.0
    if len(shape) == 1:
        return float(shape[0]), float(shape[0])
    rf = float(np.prod(shape[:-2])) if len(shape) > 2 else 1.0
    return shape[-2] * rf, shape[-1] * rf


def variance_scaling(scale, mode, distribution):
    def init(key, shape, dtype=None):
        fi, fo = _fans(shape)
        den = {"fan_in": fi, "fan_out": fo, "fan_avg": (fi + fo) / 2}[mode]
        var = scale / max(den, 1.0)
        if distribution == "uniform":
            lim = np.sqrt(3 * var)
            return _jr.uniform(key, shape, minval=-lim, maxval=lim).astype(_dt(dtype))
        return (_jr.normal(key, shape) * np.sqrt(var)).astype(_dt(dtype))
    return init


def lecun_normal():
    return variance_scaling(1.0, "fan_in", "normal")


def xavier_normal():
    return variance_scaling(1.0, "fan_avg", "normal")


glorot_normal = xavier_normal


def xavier_uniform():
    return variance_scaling(1.0, "fan_avg", "uniform")


glorot_uniform = xavier_uniform


def he_normal():
    return variance_scaling(2.0, "fan_in", "normal")


kaiming_normal = he_normal
