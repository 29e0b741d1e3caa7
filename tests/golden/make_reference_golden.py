"""Writes tests/golden/ref/<case>.npz by running the reference's OWN model files (unmodified,
imported from the checkout CSSM_REFERENCE_ROOT names, default /root/reference) on the NumPy
stand-ins for jax / flax.linen under oracle/_shim, in double precision.

    python -m tests.golden.make_reference_golden [case-name ...]

For each case of tests/golden/ref_cases.py: the reference module is constructed with the case's
arguments, `init` gives the parameter tree (so names and shapes are the reference's), every
leaf is perturbed and rounded to float32 (non-zero biases; the library and the reference then see
identical values), `apply` gives the output.  The fixture stores the parameters (float32), the
BatchNorm statistics where the model has them, and the output (float64; at 32768 seeded
positions when it is larger)."""
from __future__ import annotations

import os
import sys

import numpy as np

from oracle import ref_loader
from tests.golden import ref_cases as rc

_MODULE_OF = {"SimpleCSSM": "simple_cssm", "CSSMSHViT": "cssm_shvit", "CSSMSHViTBlock": "cssm_shvit"}


def perturb(tree, rng, case, path=""):
    """float32-exact parameters: biases and other 1-D leaves get N(0, 0.3^2) added (0.03 on the
    block's last projection so that the signal dominates the output), LayerNorm / RMS scales
    N(0, 0.2^2), kernels are kept; a block's spectral kernel can be scaled up so that |K_hat| is
    not negligible."""
    out = {}
    for k, v in tree.items():
        p = path + "/" + k
        if isinstance(v, dict):
            out[k] = perturb(v, rng, case, p)
            continue
        v = np.asarray(v, np.float64)
        last = any(s in p for s in ("/out_proj/", "/output_proj/", "/head/"))
        if k == "bias":
            v = v + (0.03 if last else 0.3) * rng.standard_normal(v.shape)
        elif k in ("scale", "rms_scale"):
            v = v + 0.2 * rng.standard_normal(v.shape)
        elif v.ndim == 1:
            v = v + 0.3 * rng.standard_normal(v.shape)
        elif k == "kernel" and v.ndim == 3 and "spectral_scale" in case:
            v = v * case["spectral_scale"]
        out[k] = v.astype(np.float32)
    return out


def perturb_stats(tree, rng):
    out = {}
    for k, v in tree.items():
        if isinstance(v, dict):
            out[k] = perturb_stats(v, rng)
        elif k == "var":
            out[k] = (np.asarray(v) * np.exp(0.3 * rng.standard_normal(np.shape(v)))).astype(np.float32)
        else:
            out[k] = (np.asarray(v) + 0.2 * rng.standard_normal(np.shape(v))).astype(np.float32)
    return out


def widen(tree):
    return {k: widen(v) if isinstance(v, dict) else np.asarray(v, np.float64) for k, v in tree.items()}


def run_reference(case, params=None, stats=None):
    """-> (params float32, stats float32 or None, output float64).  With params=None the tree
    comes from the reference's own init (perturbed)."""
    mod = ref_loader.load(_MODULE_OF.get(case["ref_class"], "cssm"))
    import jax                     # the stand-in: ref_loader.load put it on sys.path
    kwargs = dict(case["ref_kwargs"])
    if "dtype" in kwargs:
        import jax.numpy as jnp
        kwargs["dtype"] = {"float32": jnp.float32, "bfloat16": jnp.bfloat16}[kwargs["dtype"]]
    module = getattr(mod, case["ref_class"])(**kwargs)
    x = rc.make_input(case).astype(np.float64)
    call_kw = case.get("call_kwargs", {})
    if params is None and "seeded_params" in case:
        params, stats = rc.seeded_params(case)
        tree = module.init(jax.random.PRNGKey(0), x[:1], **call_kw)
        shapes = lambda t: {k: v.shape for k, v in rc.flatten(t).items()}
        assert shapes(tree["params"]) == shapes(params), "seeded tree differs from the reference's"
        assert shapes(tree["batch_stats"]) == shapes(stats)
    elif params is None:
        variables = module.init(jax.random.PRNGKey(case["seed"]), x, **call_kw)
        rng = np.random.default_rng(case["seed"] + 7)
        params = perturb(variables["params"], rng, case)
        stats = perturb_stats(variables["batch_stats"], rng) if "batch_stats" in variables else None
    variables = {"params": widen(params)}
    if stats is not None:
        variables["batch_stats"] = widen(stats)
    y = module.apply(variables, x, **call_kw)
    return params, stats, np.asarray(y, np.float64)


def write_case(case):
    params, stats, y = run_reference(case)
    pos = rc.stored_positions(case["name"], y.size)
    arrays = {}
    if "seeded_params" not in case:
        arrays = {"p:" + k: v for k, v in rc.flatten(params).items()}
    if stats is not None and "seeded_params" not in case:
        arrays.update({"s:" + k: v for k, v in rc.flatten(stats).items()})
    arrays["y"] = rc.pick(y, pos)
    arrays["y_shape"] = np.asarray(y.shape)
    if pos is not None:
        arrays["positions"] = pos
    os.makedirs(rc.REF_DIR, exist_ok=True)
    path = os.path.join(rc.REF_DIR, case["name"] + ".npz")
    np.savez_compressed(path, **arrays)
    return path, y


def main(argv):
    names = argv or [c["name"] for c in rc.CASES]
    for n in names:
        path, y = write_case(rc.BY_NAME[n])
        sig = np.linalg.norm(y - y.mean()) / max(np.linalg.norm(y), 1e-30)
        print(f"{n:42s} out{tuple(y.shape)}  variation/norm={sig:.3f}  {os.path.getsize(path) / 1024:.0f} KB")


if __name__ == "__main__":
    main(sys.argv[1:])
