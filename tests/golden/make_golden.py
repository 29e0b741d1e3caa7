"""Generates the golden vectors under tests/golden/ from the NumPy oracle (fp64 tier).

The reference implementation needs JAX/Flax, which cannot be installed where this repository
is built, so these vectors come from the oracle itself: they pin it against drift and give the
GPU tests committed inputs/outputs to compare with.  Run:  python -m tests.golden.make_golden
"""
import os

import numpy as np

from oracle import cssm_oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))


def gated_case():
    B, T, H, W, C, ks = 2, 3, 8, 8, 8, 5
    x = np.random.default_rng(11).standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_gated_params(12, C, H, W, kernel_size=ks, gate_type="factored", bias_scale=0.1)
    kw = dict(kernel_size=ks, rope_mode="spatiotemporal", gate_type="factored")
    return x, p, kw


def gated_case_64():
    B, T, H, W, C, ks = 1, 2, 64, 64, 4, 11
    x = np.random.default_rng(21).standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_gated_params(22, C, H, W, kernel_size=ks, gate_type="factored", bias_scale=0.1)
    kw = dict(kernel_size=ks, rope_mode="spatiotemporal", gate_type="factored")
    return x, p, kw


def gdn_case():
    B, T, H, W, C, ks = 2, 3, 8, 8, 8, 5
    x = np.random.default_rng(31).standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_gdn_params(32, C, H, W, delta_key_dim=4, kernel_size=ks, gate_type="factored",
                            qkv_conv_size=5, bias_scale=0.1, perturb_rms=True)
    kw = dict(delta_key_dim=4, kernel_size=ks, rope_mode="mrope", gate_type="factored",
              qkv_conv_size=5)
    return x, p, kw


def main():
    x, p, kw = gated_case()
    np.savez_compressed(os.path.join(HERE, "gated_small.npz"), x=x,
                        y=orc.gated_forward(p, x, **kw).astype(np.float64))
    x, p, kw = gated_case_64()
    np.savez_compressed(os.path.join(HERE, "gated_64.npz"), x=x,
                        y=orc.gated_forward(p, x, **kw).astype(np.float32))
    x, p, kw = gdn_case()
    np.savez_compressed(os.path.join(HERE, "gdn_small.npz"), x=x,
                        y=orc.gdn_forward(p, x, **kw).astype(np.float64))


if __name__ == "__main__":
    main()
