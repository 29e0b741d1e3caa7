"""`jax.nn` activations on NumPy arrays (same formulas as the JAX definitions)."""
from __future__ import annotations

import numpy as np


def sigmoid(x):
    x = np.asarray(x)
    z = np.exp(-np.abs(x))
    return np.where(x >= 0, 1.0 / (1.0 + z), z / (1.0 + z)).astype(x.dtype)


def silu(x):
    return x * sigmoid(x)


swish = silu


def softplus(x):
    x = np.asarray(x)
    return np.logaddexp(x, 0.0).astype(x.dtype)


def relu(x):
    return np.maximum(x, 0)


def tanh(x):
    return np.tanh(x)


def gelu(x, approximate=True):
    """jax.nn.gelu: the tanh form unless approximate=False."""
    x = np.asarray(x)
    if approximate:
        xf = x.astype(np.float64) if x.dtype.itemsize < 8 and x.dtype.kind == "f" else x
        c = np.sqrt(2.0 / np.pi)
        y = 0.5 * xf * (1.0 + np.tanh(c * (xf + 0.044715 * xf ** 3)))
        return y.astype(x.dtype)
    from scipy.special import erf
    return (0.5 * x * (1.0 + erf(x / np.sqrt(2.0)))).astype(x.dtype)


def softmax(x, axis=-1):
    m = np.max(x, axis=axis, keepdims=True)
    e = np.exp(x - m)
    return e / np.sum(e, axis=axis, keepdims=True)
