"""`jax.lax` stand-in: the few structured primitives the reference's model files call."""
from __future__ import annotations

import numpy as np


def rsqrt(x):
    return 1.0 / np.sqrt(x)


def stop_gradient(x):
    return x


def _sl(a, axis, s):
    idx = [slice(None)] * a.ndim
    idx[axis] = s
    return a[tuple(idx)]


def _interleave(a, b, axis):
    """a[0], b[0], a[1], b[1], ... along axis (a has as many or one more element than b)."""
    na, nb = a.shape[axis], b.shape[axis]
    shape = list(a.shape)
    shape[axis] = na + nb
    out = np.empty(shape, dtype=np.result_type(a, b))
    _sl(out, axis, slice(0, None, 2))[...] = a
    _sl(out, axis, slice(1, None, 2))[...] = b
    return out


def associative_scan(fn, elems, reverse=False, axis=0):
    """Inclusive scan with the recursive odd/even schedule of `jax.lax.associative_scan`:
    combine adjacent pairs, scan the half-length sequence of pair results (these are the odd
    positions), then fill the even positions with one more combine.  `fn(a, b)` receives the
    earlier elements as `a` and the later ones as `b`, slices stacked along `axis`."""
    is_tuple = isinstance(elems, (tuple, list))
    flat = list(elems) if is_tuple else [elems]
    flat = [np.asarray(e) for e in flat]
    axis = axis % flat[0].ndim
    if reverse:
        flat = [np.flip(e, axis) for e in flat]

    def comb(a, b):
        r = fn(tuple(a), tuple(b)) if is_tuple else fn(a[0], b[0])
        return list(r) if is_tuple else [r]

    def scan(el):
        n = el[0].shape[axis]
        if n < 2:
            return el
        reduced = comb([_sl(e, axis, slice(0, n - 1, 2)) for e in el],
                       [_sl(e, axis, slice(1, None, 2)) for e in el])
        odd = scan(reduced)
        if n % 2 == 0:
            even = comb([_sl(e, axis, slice(0, -1)) for e in odd],
                        [_sl(e, axis, slice(2, None, 2)) for e in el])
        else:
            even = comb(odd, [_sl(e, axis, slice(2, None, 2)) for e in el])
        even = [np.concatenate([_sl(e, axis, slice(0, 1)), r], axis=axis) for e, r in zip(el, even)]
        return [_interleave(ev, od, axis) for ev, od in zip(even, odd)]

    out = scan(flat)
    if reverse:
        out = [np.flip(o, axis) for o in out]
    return tuple(out) if is_tuple else out[0]


def _tree_index(tree, i):
    if tree is None:
        return None
    if isinstance(tree, (tuple, list)):
        return type(tree)(_tree_index(t, i) for t in tree)
    return tree[i]


def _tree_stack(items):
    first = items[0]
    if first is None:
        return None
    if isinstance(first, (tuple, list)):
        return type(first)(_tree_stack([it[j] for it in items]) for j in range(len(first)))
    return np.stack(items)


def _tree_len(tree):
    if isinstance(tree, (tuple, list)):
        for t in tree:
            n = _tree_len(t)
            if n is not None:
                return n
        return None
    return None if tree is None else tree.shape[0]


def scan(f, init, xs, length=None, reverse=False, unroll=1):
    n = length if xs is None else _tree_len(xs)
    order = range(n - 1, -1, -1) if reverse else range(n)
    carry, ys = init, [None] * n
    for i in order:
        carry, y = f(carry, _tree_index(xs, i))
        ys[i] = y
    return carry, _tree_stack(ys)


def conv_general_dilated(*a, **k):  # pragma: no cover
    raise NotImplementedError("conv_general_dilated is outside the covered paths")
