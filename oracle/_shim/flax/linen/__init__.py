"""`flax.linen` stand-in on NumPy: Module scoping with a nested variable dict, and the layers the
reference's model files instantiate (Dense, Conv, LayerNorm, BatchNorm, GroupNorm, Dropout,
max_pool / avg_pool).  Parameter names, shapes and auto-naming (`ClassName_<n>`) follow Flax so
that a tree produced by `init` here has the layout of a real Flax checkpoint."""
from __future__ import annotations

import dataclasses
import functools
from typing import Any, Optional

import numpy as np

from jax import nn as _jnn
from jax import random as _jr

from . import initializers  # noqa: F401

sigmoid = _jnn.sigmoid
silu = _jnn.silu
swish = _jnn.silu
softplus = _jnn.softplus
gelu = _jnn.gelu
relu = _jnn.relu
softmax = _jnn.softmax
tanh = _jnn.tanh

_STACK: list = []          # modules whose compact method is running (innermost last)


class _Root:
    """State of one init/apply call: variable collections, mutability, rng streams."""

    def __init__(self, variables, initializing, mutable, rngs):
        self.variables = variables
        self.initializing = initializing
        self.mutable = mutable
        self.rngs = rngs or {}
        self.rng_count = {}


def _is_mutable(root, col):
    m = root.mutable
    if m is True:
        return True
    if not m:
        return False
    return col in m


def compact(fn):
    @functools.wraps(fn)
    def wrapped(self, *a, **k):
        if self._root is None:
            raise RuntimeError(f"{type(self).__name__} called outside init/apply")
        _STACK.append(self)
        object.__setattr__(self, "_auto", {})
        try:
            return fn(self, *a, **k)
        finally:
            _STACK.pop()
    wrapped._compact = True
    return wrapped


class Module:
    name: Optional[str] = None
    parent: Any = None

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        ann = dict(cls.__dict__.get("__annotations__", {}))
        ann.pop("name", None)
        ann.pop("parent", None)
        ann["parent"] = Any
        ann["name"] = Optional[str]
        cls.__annotations__ = ann
        cls.parent = dataclasses.field(default=None, kw_only=True)
        cls.name = dataclasses.field(default=None, kw_only=True)
        dataclasses.dataclass(cls, eq=False, repr=False)

    def __post_init__(self):
        object.__setattr__(self, "_root", None)
        object.__setattr__(self, "_path", ())
        object.__setattr__(self, "_auto", {})
        if _STACK:
            par = _STACK[-1]
            nm = self.name
            if nm is None:
                base = type(self).__name__
                idx = par._auto.get(base, 0)
                par._auto[base] = idx + 1
                nm = f"{base}_{idx}"
                object.__setattr__(self, "name", nm)
            object.__setattr__(self, "parent", par)
            object.__setattr__(self, "_root", par._root)
            object.__setattr__(self, "_path", par._path + (nm,))

    # ----------------------------------------------------------------- variables
    def _col(self, col, create):
        node = self._root.variables.get(col)
        if node is None:
            if not create:
                return None
            node = self._root.variables.setdefault(col, {})
        for p in self._path:
            nxt = node.get(p)
            if nxt is None:
                if not create:
                    return None
                nxt = node.setdefault(p, {})
            node = nxt
        return node

    def param(self, name, init_fn, *init_args, **init_kw):
        node = self._col("params", self._root.initializing)
        if node is not None and name in node:
            return np.asarray(node[name])
        if not self._root.initializing:
            raise KeyError(f"missing parameter {'/'.join(self._path + (name,))}")
        val = np.asarray(init_fn(self.make_rng("params"), *init_args, **init_kw))
        node[name] = val
        return val

    def variable(self, col, name, init_fn=None, *init_args):
        node = self._col(col, self._root.initializing or _is_mutable(self._root, col))
        if node is None or name not in node:
            if node is None:
                raise KeyError(f"missing variable {col}/{'/'.join(self._path + (name,))}")
            node[name] = init_fn(*init_args)
        return _Var(node, name)

    def has_variable(self, col, name):
        node = self._col(col, False)
        return node is not None and name in node

    def sow(self, col, name, value, **kw):
        if not (self._root.initializing or _is_mutable(self._root, col)):
            return False
        node = self._col(col, True)
        node[name] = tuple(node.get(name, ())) + (value,)
        return True

    def make_rng(self, stream="params"):
        root = self._root
        base = root.rngs.get(stream)
        if base is None:
            raise KeyError(f"no rng stream '{stream}' was given")
        n = root.rng_count.get(stream, 0)
        root.rng_count[stream] = n + 1
        return _jr.fold_in(base, n)

    def is_initializing(self):
        return self._root.initializing

    def is_mutable_collection(self, col):
        return self._root.initializing or _is_mutable(self._root, col)

    # ----------------------------------------------------------------- entry points
    def _run(self, root, method, args, kwargs):
        object.__setattr__(self, "_root", root)
        object.__setattr__(self, "_path", ())
        try:
            fn = getattr(self, method) if isinstance(method, str) else functools.partial(method, self)
            return fn(*args, **kwargs)
        finally:
            object.__setattr__(self, "_root", None)

    def init(self, rngs, *args, method="__call__", **kwargs):
        if not isinstance(rngs, dict):
            rngs = {"params": rngs}
        root = _Root({}, True, True, rngs)
        self._run(root, method, args, kwargs)
        return root.variables

    def init_with_output(self, rngs, *args, method="__call__", **kwargs):
        if not isinstance(rngs, dict):
            rngs = {"params": rngs}
        root = _Root({}, True, True, rngs)
        out = self._run(root, method, args, kwargs)
        return out, root.variables

    def apply(self, variables, *args, rngs=None, mutable=False, method="__call__", **kwargs):
        if rngs is not None and not isinstance(rngs, dict):
            rngs = {"params": rngs}
        vars_ = {k: v for k, v in variables.items()}
        root = _Root(vars_, False, mutable, rngs)
        out = self._run(root, method, args, kwargs)
        if mutable:
            cols = vars_.keys() if mutable is True else mutable
            return out, {c: vars_[c] for c in cols if c in vars_ and c != "params"}
        return out


class _Var:
    def __init__(self, node, name):
        self._node, self._name = node, name

    @property
    def value(self):
        return self._node[self._name]

    @value.setter
    def value(self, v):
        self._node[self._name] = v


# --------------------------------------------------------------------------- layers
def _promote(dtype, *arrays):
    """Flax's promote_dtype: cast every array to `dtype`, or to their common type if None."""
    arrays = [np.asarray(a) for a in arrays]
    if dtype is None:
        dtype = np.result_type(*[a.dtype for a in arrays])
    return [a.astype(dtype) for a in arrays], np.dtype(dtype)


def _acc(a):
    """Low-precision operands are multiplied in float32 (as XLA accumulates) and rounded after."""
    return a.astype(np.float32) if a.dtype.itemsize < 4 else a


class Dense(Module):
    features: int = 0
    use_bias: bool = True
    dtype: Any = None
    param_dtype: Any = None
    kernel_init: Any = None
    bias_init: Any = None
    precision: Any = None

    @compact
    def __call__(self, x):
        import jax.numpy as jnp
        pd = self.param_dtype or jnp.float32
        k = self.param("kernel", self.kernel_init or initializers.lecun_normal(),
                       (x.shape[-1], self.features), pd)
        b = self.param("bias", self.bias_init or initializers.zeros, (self.features,), pd) \
            if self.use_bias else None
        (x, k), dt = _promote(self.dtype, x, k)
        y = (_acc(x) @ _acc(k))
        if b is not None:
            y = y + _acc(b.astype(dt))
        return y.astype(dt)


def _pad_amounts(padding, in_size, k, stride, dil=1):
    if isinstance(padding, str):
        if padding == "VALID":
            return [(0, 0)] * len(in_size)
        if padding == "SAME":
            out = []
            for n, kk, s in zip(in_size, k, stride):
                o = -(-n // s)
                tot = max((o - 1) * s + (kk - 1) * dil + 1 - n, 0)
                out.append((tot // 2, tot - tot // 2))
            return out
        raise NotImplementedError(padding)
    if isinstance(padding, int):
        return [(padding, padding)] * len(in_size)
    return [tuple(p) if not isinstance(p, int) else (p, p) for p in padding]


class Conv(Module):
    features: int = 0
    kernel_size: Any = ()
    strides: Any = 1
    padding: Any = "SAME"
    input_dilation: Any = 1
    kernel_dilation: Any = 1
    feature_group_count: int = 1
    use_bias: bool = True
    dtype: Any = None
    param_dtype: Any = None
    kernel_init: Any = None
    bias_init: Any = None
    precision: Any = None

    @compact
    def __call__(self, x):
        import jax.numpy as jnp
        ks = (self.kernel_size,) if isinstance(self.kernel_size, int) else tuple(self.kernel_size)
        nd = len(ks)
        st = (self.strides,) * nd if isinstance(self.strides, int) or self.strides is None \
            else tuple(self.strides)
        if self.strides is None:
            st = (1,) * nd
        cin = x.shape[-1]
        g = self.feature_group_count
        pd = self.param_dtype or jnp.float32
        k = self.param("kernel", self.kernel_init or initializers.lecun_normal(),
                       ks + (cin // g, self.features), pd)
        b = self.param("bias", self.bias_init or initializers.zeros, (self.features,), pd) \
            if self.use_bias else None
        (x, k), dt = _promote(self.dtype, x, k)
        lead = x.shape[:-(nd + 1)]
        xs = _acc(x).reshape((-1,) + x.shape[-(nd + 1):])
        pads = _pad_amounts(self.padding, xs.shape[1:1 + nd], ks, st)
        xs = np.pad(xs, [(0, 0)] + list(pads) + [(0, 0)])
        outsz = [(xs.shape[1 + d] - ks[d]) // st[d] + 1 for d in range(nd)]
        kf = _acc(k)
        cog = self.features // g
        y = np.zeros((xs.shape[0],) + tuple(outsz) + (self.features,), dtype=np.result_type(xs, kf))
        for tap in np.ndindex(*ks):
            sl = (slice(None),) + tuple(slice(tap[d], tap[d] + (outsz[d] - 1) * st[d] + 1, st[d])
                                        for d in range(nd))
            xt = xs[sl]                                            # (N, *out, cin)
            w = kf[tap]                                            # (cin/g, features)
            if g == 1:
                y += xt @ w
            elif cin == g:                                         # depthwise (multiplier cog)
                y += np.repeat(xt, cog, axis=-1) * w[0]
            else:
                xg = xt.reshape(xt.shape[:-1] + (g, cin // g))
                wg = w.reshape(cin // g, g, cog)
                y += np.einsum("...gi,igo->...go", xg, wg).reshape(y.shape)
        if b is not None:
            y = y + _acc(b.astype(dt))
        return y.reshape(lead + y.shape[1:]).astype(dt)


def _canon_axes(ndim, axes):
    if isinstance(axes, int):
        axes = (axes,)
    return tuple(sorted(a % ndim for a in axes))


def _moments(x, axes, fast=True):
    xf = x.astype(np.float32) if x.dtype.itemsize < 4 else x
    mean = xf.mean(axis=axes, keepdims=True)
    if fast:
        var = np.maximum((xf * xf).mean(axis=axes, keepdims=True) - mean * mean, 0.0)
    else:
        var = ((xf - mean) ** 2).mean(axis=axes, keepdims=True)
    return xf, mean, var


class LayerNorm(Module):
    epsilon: float = 1e-6
    dtype: Any = None
    param_dtype: Any = None
    use_bias: bool = True
    use_scale: bool = True
    bias_init: Any = None
    scale_init: Any = None
    reduction_axes: Any = -1
    feature_axes: Any = -1
    use_fast_variance: bool = True

    @compact
    def __call__(self, x):
        import jax.numpy as jnp
        x = np.asarray(x)
        red = _canon_axes(x.ndim, self.reduction_axes)
        feat = _canon_axes(x.ndim, self.feature_axes)
        pd = self.param_dtype or jnp.float32
        fshape = tuple(x.shape[a] for a in feat)
        bshape = [1] * x.ndim
        for a in feat:
            bshape[a] = x.shape[a]
        xf, mean, var = _moments(x, red, self.use_fast_variance)
        y = (xf - mean) / np.sqrt(var + self.epsilon)
        args = [x]
        if self.use_scale:
            s = self.param("scale", self.scale_init or initializers.ones, fshape, pd)
            y = y * s.reshape(bshape)
            args.append(s)
        if self.use_bias:
            b = self.param("bias", self.bias_init or initializers.zeros, fshape, pd)
            y = y + b.reshape(bshape)
            args.append(b)
        dt = self.dtype or np.result_type(*[np.asarray(a).dtype for a in args])
        return y.astype(dt)


class GroupNorm(Module):
    num_groups: Optional[int] = 32
    group_size: Optional[int] = None
    epsilon: float = 1e-6
    dtype: Any = None
    param_dtype: Any = None
    use_bias: bool = True
    use_scale: bool = True

    @compact
    def __call__(self, x):
        import jax.numpy as jnp
        x = np.asarray(x)
        C = x.shape[-1]
        G = self.num_groups if self.num_groups is not None else C // self.group_size
        pd = self.param_dtype or jnp.float32
        xg = x.reshape(x.shape[:-1] + (G, C // G))
        red = tuple(range(1, x.ndim - 1)) + (x.ndim,)
        xf, mean, var = _moments(xg, red)
        y = ((xf - mean) / np.sqrt(var + self.epsilon)).reshape(x.shape)
        if self.use_scale:
            y = y * self.param("scale", initializers.ones, (C,), pd)
        if self.use_bias:
            y = y + self.param("bias", initializers.zeros, (C,), pd)
        return y.astype(self.dtype or x.dtype)


class BatchNorm(Module):
    use_running_average: Optional[bool] = None
    axis: int = -1
    momentum: float = 0.99
    epsilon: float = 1e-5
    dtype: Any = None
    param_dtype: Any = None
    use_bias: bool = True
    use_scale: bool = True
    axis_name: Any = None

    @compact
    def __call__(self, x, use_running_average=None):
        import jax.numpy as jnp
        x = np.asarray(x)
        ura = self.use_running_average if use_running_average is None else use_running_average
        C = x.shape[-1]
        pd = self.param_dtype or jnp.float32
        ra_mean = self.variable("batch_stats", "mean", lambda: np.zeros((C,), pd))
        ra_var = self.variable("batch_stats", "var", lambda: np.ones((C,), pd))
        red = tuple(range(x.ndim - 1))
        xf = x.astype(np.float32) if x.dtype.itemsize < 4 else x
        if ura:
            mean, var = np.asarray(ra_mean.value), np.asarray(ra_var.value)
        else:
            mean = xf.mean(axis=red)
            var = np.maximum((xf * xf).mean(axis=red) - mean * mean, 0.0)
            if not self._root.initializing and _is_mutable(self._root, "batch_stats"):
                ra_mean.value = self.momentum * ra_mean.value + (1 - self.momentum) * mean
                ra_var.value = self.momentum * ra_var.value + (1 - self.momentum) * var
        y = (xf - mean) / np.sqrt(var + self.epsilon)
        if self.use_scale:
            y = y * self.param("scale", initializers.ones, (C,), pd)
        if self.use_bias:
            y = y + self.param("bias", initializers.zeros, (C,), pd)
        return y.astype(self.dtype or x.dtype)


class Dropout(Module):
    rate: float = 0.0
    deterministic: Optional[bool] = None

    @compact
    def __call__(self, x, deterministic=None):
        det = self.deterministic if deterministic is None else deterministic
        if det or self.rate == 0.0:
            return x
        keep = 1.0 - self.rate
        mask = _jr.bernoulli(self.make_rng("dropout"), keep, x.shape)
        return np.where(mask, x / keep, 0).astype(x.dtype)


def _pool(x, window_shape, strides, padding, init, op):
    x = np.asarray(x)
    nd = len(window_shape)
    strides = tuple(strides) if strides is not None else (1,) * nd
    lead = x.shape[:-(nd + 1)]
    xs = x.reshape((-1,) + x.shape[-(nd + 1):])
    pads = _pad_amounts(padding, xs.shape[1:1 + nd], window_shape, strides)
    xs = np.pad(xs, [(0, 0)] + list(pads) + [(0, 0)], constant_values=init)
    outsz = [(xs.shape[1 + d] - window_shape[d]) // strides[d] + 1 for d in range(nd)]
    y = None
    for tap in np.ndindex(*window_shape):
        sl = (slice(None),) + tuple(slice(tap[d], tap[d] + (outsz[d] - 1) * strides[d] + 1, strides[d])
                                    for d in range(nd))
        y = xs[sl] if y is None else op(y, xs[sl])
    return y.reshape(lead + y.shape[1:])


def max_pool(x, window_shape, strides=None, padding="VALID"):
    return _pool(x, window_shape, strides, padding, -np.inf, np.maximum)


def avg_pool(x, window_shape, strides=None, padding="VALID", count_include_pad=True):
    if not count_include_pad:
        raise NotImplementedError
    return _pool(x, window_shape, strides, padding, 0.0, np.add) / float(np.prod(window_shape))
