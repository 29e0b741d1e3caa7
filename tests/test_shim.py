"""The NumPy stand-ins under oracle/_shim against independent implementations: layers against
torch.nn.functional, the associative scan against a sequential fold (non-commutative operator,
odd and even lengths), lax.scan, and Flax's parameter naming."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F

_SHIM = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_shim")


@pytest.fixture(scope="module")
def shim():
    if _SHIM not in sys.path:
        sys.path.insert(0, _SHIM)
    import jax
    import flax.linen as nn
    assert jax.__file__.startswith(_SHIM)
    return jax, nn


def _rng():
    return np.random.default_rng(0)


def _apply(mod, params, x, **kw):
    return mod.apply({"params": params}, x, **kw)


@pytest.mark.parametrize("k,stride,groups,pad", [(3, 1, 1, "SAME"), (3, 2, 1, "SAME"), (7, 1, 6, "SAME"),
                                                 (3, 1, 6, "SAME"), (5, 1, 6, "SAME"), (1, 1, 1, "SAME"),
                                                 (4, 1, 1, "VALID"), (3, 2, 2, "SAME")])
@pytest.mark.parametrize("hw", [(9, 8), (14, 14)])
def test_conv2d_matches_torch(shim, k, stride, groups, pad, hw):
    jax, nn = shim
    r = _rng()
    cin, cout = 6, 12 if groups < 6 else 6
    x = r.standard_normal((2,) + hw + (cin,))
    w = r.standard_normal((k, k, cin // groups, cout))
    b = r.standard_normal(cout)
    y = _apply(nn.Conv(cout, kernel_size=(k, k), strides=(stride, stride), padding=pad,
                       feature_group_count=groups), {"kernel": w, "bias": b}, x)
    xt = torch.from_numpy(x).permute(0, 3, 1, 2)
    if pad == "SAME":                   # XLA's SAME: total = (ceil(n/s)-1)*s + k - n, low half first
        pads = []
        for n in hw[::-1]:
            tot = max((-(-n // stride) - 1) * stride + k - n, 0)
            pads += [tot // 2, tot - tot // 2]
        xt = F.pad(xt, pads)
    ref = F.conv2d(xt, torch.from_numpy(w).permute(3, 2, 0, 1), torch.from_numpy(b),
                   stride=stride, groups=groups).permute(0, 2, 3, 1).numpy()
    assert y.shape == ref.shape
    assert np.abs(y - ref).max() < 1e-12


def test_conv1d_causal_matches_torch(shim):
    jax, nn = shim
    r = _rng()
    x = r.standard_normal((5, 7, 4))
    w = r.standard_normal((4, 1, 4))
    b = r.standard_normal(4)
    xp = np.pad(x, ((0, 0), (3, 0), (0, 0)))
    y = _apply(nn.Conv(4, kernel_size=(4,), feature_group_count=4, padding="VALID"),
               {"kernel": w, "bias": b}, xp)
    ref = F.conv1d(torch.from_numpy(xp).permute(0, 2, 1), torch.from_numpy(w).permute(2, 1, 0),
                   torch.from_numpy(b), groups=4).permute(0, 2, 1).numpy()
    assert np.abs(y - ref).max() < 1e-12


def test_dense_layernorm_batchnorm_pool_gelu(shim):
    jax, nn = shim
    r = _rng()
    x = r.standard_normal((3, 6, 5, 8))
    w, b = r.standard_normal((8, 4)), r.standard_normal(4)
    assert np.abs(_apply(nn.Dense(4), {"kernel": w, "bias": b}, x) - (x @ w + b)).max() < 1e-12
    s, bb = r.standard_normal(8), r.standard_normal(8)
    y = _apply(nn.LayerNorm(), {"scale": s, "bias": bb}, x)
    ref = F.layer_norm(torch.from_numpy(x), (8,), torch.from_numpy(s), torch.from_numpy(bb), eps=1e-6)
    assert np.abs(y - ref.numpy()).max() < 1e-10
    y = _apply(nn.LayerNorm(reduction_axes=(1, 2, 3), feature_axes=-1), {"scale": s, "bias": bb}, x)
    xn = F.layer_norm(torch.from_numpy(x), x.shape[1:], eps=1e-6).numpy()
    assert np.abs(y - (xn * s + bb)).max() < 1e-10
    mean, var = r.standard_normal(8), r.random(8) + 0.5
    y = nn.BatchNorm(use_running_average=True).apply(
        {"params": {"scale": s, "bias": bb}, "batch_stats": {"mean": mean, "var": var}}, x)
    ref = F.batch_norm(torch.from_numpy(x).permute(0, 3, 1, 2), torch.from_numpy(mean),
                       torch.from_numpy(var), torch.from_numpy(s), torch.from_numpy(bb),
                       training=False, eps=1e-5).permute(0, 2, 3, 1).numpy()
    assert np.abs(y - ref).max() < 1e-10
    xo = r.standard_normal((2, 7, 9, 3))
    y = nn.max_pool(xo, (2, 2), strides=(2, 2), padding="SAME")
    ref = F.max_pool2d(F.pad(torch.from_numpy(xo).permute(0, 3, 1, 2), (0, 1, 0, 1), value=-np.inf), 2
                       ).permute(0, 2, 3, 1).numpy()
    assert np.array_equal(y, ref)
    g = jax.nn.gelu(x)
    assert np.abs(g - F.gelu(torch.from_numpy(x), approximate="tanh").numpy()).max() < 1e-12
    assert np.abs(jax.nn.silu(x) - F.silu(torch.from_numpy(x)).numpy()).max() < 1e-12
    assert np.abs(jax.nn.softplus(x) - F.softplus(torch.from_numpy(x)).numpy()).max() < 1e-12


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 8, 13, 32])
def test_associative_scan_matches_sequential_fold(shim, n):
    jax, nn = shim
    r = _rng()
    M = 0.5 * r.standard_normal((2, n, 3, 3))
    u = r.standard_normal((2, n, 3))

    def op(a, b):                      # affine maps: later after earlier (not commutative)
        Ma, ua = a
        Mb, ub = b
        return Mb @ Ma, np.einsum("...ij,...j->...i", Mb, ua) + ub

    Ms, us = jax.lax.associative_scan(op, (M, u), axis=1)
    Mc, uc = M[:, 0], u[:, 0]
    for t in range(n):
        if t:
            Mc, uc = op((Mc, uc), (M[:, t], u[:, t]))
        assert np.abs(Ms[:, t] - Mc).max() < 1e-10 and np.abs(us[:, t] - uc).max() < 1e-10


def test_lax_scan(shim):
    jax, nn = shim
    xs = np.arange(12.0).reshape(6, 2)
    carry, ys = jax.lax.scan(lambda c, x: (c + x, c * 2), np.zeros(2), xs)
    assert np.array_equal(carry, xs.sum(0))
    assert np.array_equal(ys, 2 * (np.cumsum(xs, 0) - xs))


def test_auto_names_follow_flax(shim):
    jax, nn = shim

    class Inner(nn.Module):
        n: int

        @nn.compact
        def __call__(self, x):
            return nn.Dense(self.n)(x)

    class Outer(nn.Module):
        @nn.compact
        def __call__(self, x):
            x = Inner(3)(x)
            x = Inner(2)(x)
            x = nn.Dense(2, name="head")(x)
            return x + self.param("offset", nn.initializers.zeros, (2,))

    v = Outer().init(jax.random.PRNGKey(0), np.zeros((1, 4)))
    assert set(v["params"]) == {"Inner_0", "Inner_1", "head", "offset"}
    assert v["params"]["Inner_0"]["Dense_0"]["kernel"].shape == (4, 3)
    with pytest.raises(KeyError):
        Outer().apply({"params": {"head": v["params"]["head"]}}, np.zeros((1, 4)))
