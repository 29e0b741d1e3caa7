"""`jax.random` stand-in: keys are uint32 pairs, draws come from NumPy's PCG64 seeded by the key.

The values are NOT those of JAX's threefry generator; fixtures store the parameters they were
made with, so only determinism matters here.
"""
from __future__ import annotations

import numpy as np


def PRNGKey(seed):
    return np.array([0, int(seed) & 0xFFFFFFFF], dtype=np.uint32)


key = PRNGKey


def _rng(k):
    k = np.asarray(k, dtype=np.uint32).reshape(-1)
    return np.random.default_rng([int(v) for v in k])


def split(k, num=2):
    ss = np.random.SeedSequence([int(v) for v in np.asarray(k).reshape(-1)])
    return np.stack([c.generate_state(2, dtype=np.uint32) for c in ss.spawn(num)])


def fold_in(k, data):
    return np.random.SeedSequence([int(v) for v in np.asarray(k).reshape(-1)] + [int(data)]
                                  ).generate_state(2, dtype=np.uint32)


def normal(k, shape=(), dtype=np.float64):
    return _rng(k).standard_normal(tuple(shape)).astype(dtype)


def uniform(k, shape=(), dtype=np.float64, minval=0.0, maxval=1.0):
    return (_rng(k).random(tuple(shape)) * (maxval - minval) + minval).astype(dtype)


def bernoulli(k, p=0.5, shape=None):
    return _rng(k).random(tuple(shape) if shape is not None else np.shape(p)) < p


def truncated_normal(k, lower, upper, shape=(), dtype=np.float64):
    from scipy.stats import truncnorm
    return truncnorm.rvs(lower, upper, size=tuple(shape), random_state=_rng(k)).astype(dtype)
