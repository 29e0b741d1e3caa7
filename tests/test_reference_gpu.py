"""The CUDA path (through the C ABI) against the reference's own outputs.

tests/golden/ref/*.npz hold what the reference's unmodified model files computed in double
precision on the same seeded inputs and parameters (see tests/golden/make_reference_golden.py).
Tolerance: 1e-4 of the output's variation for the fp32 paths, 2e-2 for the bf16 paths (the
bf16-carry GDN static-image scan; the CSSM-SHViT blocks and models, which run with bfloat16
activations against the reference's double-precision result)."""
import numpy as np
import pytest
import torch

import cssm_b200
from tests.golden import ref_cases as rc

pytestmark = pytest.mark.gpu

_CASES = [c["name"] for c in rc.CASES if c.get("mirror")]


@pytest.mark.parametrize("name", _CASES)
def test_cuda_path_reproduces_reference(name):
    case = rc.BY_NAME[name]
    params, stats, y_ref, pos = rc.load(name)
    x = torch.from_numpy(rc.make_input(case)).cuda()
    cls = getattr(cssm_b200, case["mirror"])
    try:
        mod = cls(**case["mirror_kwargs"])
        variables = {"params": params}
        if stats is not None:
            variables["batch_stats"] = stats
        y = mod.apply(variables, x, **({"training": False} if case["family"] in ("simple", "shvit") else {}))
    except NotImplementedError as e:
        pytest.skip(f"no kernel for this field combination: {e}")
    got = rc.pick(y.float().cpu().numpy(), pos)
    assert np.isfinite(got).all()
    err = rc.rel_err(got, y_ref)
    assert err <= case.get("tol_gpu", 1e-4), f"{name}: {err:.3e}"
