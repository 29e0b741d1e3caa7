"""NumPy stand-in for the part of `jax` the reference's model files use (test infrastructure).

Arrays are plain `numpy.ndarray`.  Unless the environment variable CSSM_SHIM_WIDE is "0" when
this package is first imported, `jnp.float32` / `jnp.complex64` are aliases of the 64-bit /
128-bit NumPy types, so that a forward run on float64 inputs and parameters evaluates the
reference's graph in double precision (dataclass defaults such as `dtype = jnp.float32` are
evaluated when the reference's files are imported, so the choice is made once per process).
"""
from __future__ import annotations

import numpy as _np

from . import numpy  # noqa: F401  (jax.numpy)
from . import lax, nn, random  # noqa: F401

Array = _np.ndarray


class _Config:
    def __init__(self):
        self.values = {"shim_wide": True}

    def update(self, key, value):
        self.values[key] = value
        if key == "shim_wide":
            numpy._set_wide(bool(value))


config = _Config()


class custom_vjp:
    """Keeps the primal function; the backward rules are recorded and never used."""

    def __init__(self, fun, nondiff_argnums=()):
        self.fun = fun
        self.__name__ = getattr(fun, "__name__", "custom_vjp")
        self.__doc__ = fun.__doc__

    def defvjp(self, fwd, bwd, **kw):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *a, **k):
        return self.fun(*a, **k)


def jit(fun=None, **kw):
    if fun is None:
        return lambda f: f
    return fun


def vmap(fun, in_axes=0, out_axes=0):
    """Maps `fun` over axis `in_axes` of every argument by a Python loop."""
    def mapped(*args):
        axes = in_axes if isinstance(in_axes, (tuple, list)) else (in_axes,) * len(args)
        n = next(a.shape[ax] for a, ax in zip(args, axes) if ax is not None)
        outs = []
        for i in range(n):
            sl = [a if ax is None else _np.take(a, i, axis=ax) for a, ax in zip(args, axes)]
            outs.append(fun(*sl))
        if isinstance(outs[0], tuple):
            return tuple(_np.stack([o[j] for o in outs], axis=out_axes) for j in range(len(outs[0])))
        return _np.stack(outs, axis=out_axes)
    return mapped


class _TreeUtil:
    @staticmethod
    def tree_map(f, tree, *rest):
        if isinstance(tree, dict):
            return {k: _TreeUtil.tree_map(f, v, *[r[k] for r in rest]) for k, v in tree.items()}
        if isinstance(tree, (list, tuple)):
            return type(tree)(_TreeUtil.tree_map(f, v, *[r[i] for r in rest]) for i, v in enumerate(tree))
        return f(tree, *rest)

    @staticmethod
    def tree_leaves(tree):
        if isinstance(tree, dict):
            return [l for v in tree.values() for l in _TreeUtil.tree_leaves(v)]
        if isinstance(tree, (list, tuple)):
            return [l for v in tree for l in _TreeUtil.tree_leaves(v)]
        return [tree]


tree_util = _TreeUtil()
tree_map = _TreeUtil.tree_map
