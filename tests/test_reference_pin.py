"""The oracle against the reference's own code.

tests/golden/ref/*.npz were written by tests/golden/make_reference_golden.py, which imports the
reference's unmodified src/models/*.py on NumPy stand-ins for jax / flax.linen and runs them in
double precision.  Here every restatement under oracle/ must reproduce those outputs to 1e-9
(fp64 against fp64; the bf16-carry GDN static path to its own tolerance).  Where the reference
checkout is present the stored outputs are also re-derived, so a stale fixture cannot pass."""
import inspect

import numpy as np
import pytest

from oracle import cssm_oracle as orc
from oracle import ref_loader
from oracle import simple_oracle as so
from tests.golden import ref_cases as rc

TOL = 1e-9


def oracle_output(case, params, stats=None):
    x = rc.make_input(case).astype(np.float64)
    fam = case["family"]
    if fam == "simple":
        r = case["ref_kwargs"]
        return so.simple_forward(params, x, cssm_type=r["cssm_type"], seq_len=r.get("seq_len", 8),
                                 stem_mode=r.get("stem_mode", "default"),
                                 stem_layers=r.get("stem_layers", 2),
                                 pool_type=r.get("pool_type", "mean"),
                                 block_kwargs=case["block_kwargs"])
    if fam in ("shvit", "shvit_block"):
        from oracle import shvit_oracle as sv
        if fam == "shvit_block":
            return sv.cssm_block(x, params, **case["oracle_kwargs"])
        return sv.shvit_forward(params, stats, x, **case["oracle_kwargs"])
    return getattr(orc, case["oracle"])(params, x, **case["oracle_kwargs"])


@pytest.mark.parametrize("name", [c["name"] for c in rc.CASES])
def test_oracle_reproduces_reference(name):
    case = rc.BY_NAME[name]
    params, stats, y_ref, pos = rc.load(name)
    got = rc.pick(oracle_output(case, params, stats), pos)
    err = rc.rel_err(got, y_ref)
    assert err <= case.get("tol_oracle", TOL), f"{name}: {err:.3e}"


_LIVE = ["shvit_tiny_64", "shvit_block_stage2_14", "gated_rope_mrope_c8", "gdn_dense_gates", "gdn_static_T4_16", "nogate_ks3",
         "additive1_factored", "deltanet_channel", "simple_gated_cfg2"]


@pytest.mark.skipif(not ref_loader.available(), reason="no reference checkout on this machine")
@pytest.mark.parametrize("name", _LIVE)
def test_fixture_is_what_the_reference_computes(name):
    from tests.golden import make_reference_golden as mk
    case = rc.BY_NAME[name]
    params, stats, y_ref, pos = rc.load(name)
    _, _, y = mk.run_reference(case, params, stats)
    assert np.array_equal(rc.pick(y, pos), y_ref)


@pytest.mark.skipif(not ref_loader.available(), reason="no reference checkout on this machine")
def test_parameter_trees_match_the_mirrors():
    """Names and shapes of the reference's parameter tree (from its own init) are the ones the
    oracle's seeded initialisers produce, for both blocks."""
    import jax
    cssm = ref_loader.load("cssm")
    C, H, W = 8, 8, 10
    x = np.zeros((1, 2, H, W, C))
    shapes = lambda t: {k: v.shape for k, v in rc.flatten(t).items()}
    ref = cssm.GatedCSSM(channels=C, kernel_size=5, gate_type="factored").init(jax.random.PRNGKey(0), x)
    mine = orc.init_gated_params(0, C, H, W, kernel_size=5, gate_type="factored")
    assert shapes(ref["params"]) == shapes(mine)
    ref = cssm.GatedDeltaNetCSSM(channels=C, delta_key_dim=4, kernel_size=5, gate_type="factored",
                                 qkv_conv_size=5).init(jax.random.PRNGKey(0), x)
    mine = orc.init_gdn_params(0, C, H, W, delta_key_dim=4, kernel_size=5, gate_type="factored",
                               qkv_conv_size=5)
    assert shapes(ref["params"]) == shapes(mine)
