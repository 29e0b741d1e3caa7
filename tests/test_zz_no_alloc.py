"""GPU test of the entry point that allocates nothing.

Some users of the library cannot allocate device memory at call time — they run inside another
framework's step where that framework's allocator owns the GPU memory, or under a policy that
only lets them launch kernels.  `cssm_gated_forward_static` serves them from a fixed scratch
array inside the library.  This file is collected last on purpose: if it fails under `-x`,
every other test has already run."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import cssm_oracle as orc
from cssm_b200 import GatedCSSM
from cssm_b200._lib import check

pytestmark = pytest.mark.gpu


_KW = dict(kernel_size=11, rope_mode="spatiotemporal", gate_type="factored")


def _setup(seed):
    B, T, H, W, Cc = 2, 3, 64, 64, 8
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((B, T, H, W, Cc)).astype(np.float32)).cuda()
    p = orc.init_gated_params(seed + 1, Cc, H, W, kernel_size=_KW["kernel_size"],
                              gate_type="factored", bias_scale=0.1)
    bound = GatedCSSM(channels=Cc, **_KW).bind({"params": p})
    bound.params_np = p
    return bound, x


def test_static_scratch_entry_matches_workspace_entry_twice():
    """Two calls in a row (different inputs, so stale scratch contents would show) give the
    same output as the workspace entry point: same kernels, same order, so bit-equal, which
    is inside the 1e-4 rel-L2 tolerance the other GPU tests use; and both match the NumPy oracle,
    so the test stands without the other entry point."""
    bound, x1 = _setup(0)
    L = bound.L
    x2 = x1.flip(0) * 1.5 + 0.25
    d = bound.desc(tuple(x1.shape))
    pl = bound.plan(d)
    assert L.cssm_gated_workspace_bytes(C.byref(d)) <= L.cssm_static_scratch_bytes()
    st = torch.cuda.current_stream().cuda_stream
    for x in (x1, x2):
        want = bound(x)
        got = torch.empty_like(x)
        check(L.cssm_gated_forward_static(C.byref(d), C.byref(bound.w), pl.data_ptr(),
                                          x.data_ptr(), got.data_ptr(), st), "forward_static")
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert orc.rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= 1e-4
        assert torch.equal(got, want)
        ref = orc.gated_forward(bound.params_np, x.cpu().numpy(), **_KW)
        assert orc.rel_l2(got.cpu().numpy(), ref) <= 1e-4


def test_static_scratch_entry_rejects_oversize():
    bound, x = _setup(1)
    L = bound.L
    big = bound.desc((64, 8, 64, 64, 8))       # workspace 134 MB > 64 MiB
    assert L.cssm_gated_workspace_bytes(C.byref(big)) > L.cssm_static_scratch_bytes()
    rc = L.cssm_gated_forward_static(C.byref(big), C.byref(bound.w), 1, 1, 1, None)
    assert rc == 7          # CSSM_ERR_SIZE_LIMIT, before any pointer is touched
    bad = bound.desc((0, 8, 64, 64, 8))
    assert L.cssm_gated_forward_static(C.byref(bad), C.byref(bound.w), 1, 1, 1, None) == 2
