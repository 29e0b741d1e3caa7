"""Generates the golden vectors under tests/golden/ from the NumPy oracle (fp64 tier).

The reference implementation needs JAX/Flax, which cannot be installed where this repository
is built, so these vectors come from the oracle itself: they pin it against drift and give the
GPU tests committed inputs/outputs to compare with.  Run:  python -m tests.golden.make_golden
"""
import os

import numpy as np

from oracle import cssm_oracle as orc
from oracle import simple_oracle as so

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


SIMPLE_KW = dict(kernel_size=5, rope_mode="spatiotemporal", gate_type="factored", short_conv_size=4,
                 short_conv_spatial_size=3)


def simple_case():
    """SimpleCSSM (one stem layer, gated block, max-pool head) on 3 images of 16x16."""
    x = np.random.default_rng(41).random((3, 16, 16, 1)).astype(np.float32)
    p = so.init_simple_params(42, cin=1, embed_dim=8, H=8, W=8, stem_layers=1, bias_scale=0.1,
                              block_kwargs=SIMPLE_KW)
    return x, p


def nogate_case():
    B, T, H, W, C, ks = 2, 4, 8, 8, 8, 3
    rng = np.random.default_rng(51)
    x = rng.standard_normal((B, T, H, W, C)).astype(np.float32)
    p = {"kernel": (0.3 * rng.standard_normal((C, ks, ks))).astype(np.float32),
         "out_proj": {"kernel": (rng.standard_normal((C, C)) / np.sqrt(C)).astype(np.float32),
                      "bias": (0.1 * rng.standard_normal(C)).astype(np.float32)}}
    return x, p, ks


def additive1_case():
    B, T, H, W, C, ks = 2, 4, 8, 8, 8, 5
    x = np.random.default_rng(71).standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_additive1_params(72, C, H, W, kernel_size=ks, gate_type="factored", bias_scale=0.1)
    kw = dict(kernel_size=ks, gate_type="factored", rope_mode="spatiotemporal")
    return x, p, kw


def deltanet_case():
    B, T, H, W, C, ks = 2, 4, 8, 8, 8, 5
    x = np.random.default_rng(81).standard_normal((B, T, H, W, C)).astype(np.float32)
    p = orc.init_deltanet_params(82, C, H, W, kernel_size=ks, gate_type="dense", bias_scale=0.1)
    p["output_proj"]["bias"][:] = 0          # the signal is small next to a 0.1-scale bias
    kw = dict(kernel_size=ks, gate_type="dense", rope_mode="mrope")
    return x, p, kw


def gdn_static_case():
    B, H, W, C, ks, T = 2, 8, 8, 8, 5, 4
    x = np.random.default_rng(61).standard_normal((B, H, W, C)).astype(np.float32)
    p = orc.init_gdn_params(62, C, H, W, delta_key_dim=4, kernel_size=ks, gate_type="factored",
                            short_conv_size=0, qkv_conv_size=3, use_input_gates=False,
                            bias_scale=0.1, perturb_rms=True)
    kw = dict(num_timesteps=T, delta_key_dim=4, kernel_size=ks, gate_type="factored", qkv_conv_size=3)
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
    x, p = simple_case()
    np.savez_compressed(os.path.join(HERE, "simple_small.npz"), x=x,
                        y=so.simple_forward(p, x, seq_len=3, stem_layers=1, pool_type="max",
                                            block_kwargs=SIMPLE_KW).astype(np.float64))
    x, p, ks = nogate_case()
    np.savez_compressed(os.path.join(HERE, "nogate_small.npz"), x=x,
                        y=orc.nogate_forward(p, x, kernel_size=ks).astype(np.float64))
    x, p, kw = additive1_case()
    np.savez_compressed(os.path.join(HERE, "additive1_small.npz"), x=x,
                        y=orc.additive1_forward(p, x, **kw).astype(np.float64))
    x, p, kw = deltanet_case()
    np.savez_compressed(os.path.join(HERE, "deltanet_small.npz"), x=x,
                        y=orc.deltanet_forward(p, x, **kw).astype(np.float64))
    x, p, kw = gdn_static_case()
    np.savez_compressed(os.path.join(HERE, "gdn_static_small.npz"), x=x,
                        y=orc.gdn_static_forward(p, x, **kw).astype(np.float64))


if __name__ == "__main__":
    main()
