"""The BASELINE workloads at their FULL sizes on the GPU (batch 128; cfg2 / cfg3 / cfg4 of bench.py).

The NumPy oracle cannot evaluate 128 samples in seconds, so the full-size runs are checked through
properties that do not depend on the size:
  * batch independence: a few samples picked out of the full-size output equal the oracle's
    output for those samples alone (rel-L2 <= 1e-4, fp32) -- every sample of the batch goes
    through the same kernels, only its index differs;
  * causality: frames before t0 are bit-identical when the input changes at t >= t0 only;
  * the last-frame-only entry point returns the last frame of the full output;
  * determinism: two runs are bit-identical.
"""
import numpy as np
import pytest
import torch

import bench
from oracle import cssm_oracle as orc
from oracle import simple_oracle as so

pytestmark = pytest.mark.gpu
TOL = 1e-4
PICK = [0, 77, 127]          # samples compared with the oracle


def _model_and_block(workload):
    model = bench.make_model(workload)
    B = bench.WORKLOADS[workload]["B"]
    assert B == 128
    return model, B


def _block_input(model, B, T, H, W, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.randn((B, T, H, W, model.embed_dim), generator=g, device="cuda", dtype=torch.float32)


@pytest.mark.parametrize("workload,T,HW", [("cfg2", 8, 64), ("cfg3", 8, 64), ("cfg4", 32, 32)])
def test_block_at_full_size(workload, T, HW):
    model, B = _model_and_block(workload)
    blk = model.block()
    x = _block_input(model, B, T, HW, HW, seed=11)
    variables = blk.init(3, tuple(x.shape), bias_scale=0.1)
    bound = blk.bind(variables)
    y = bound(x)
    assert torch.isfinite(y).all()
    # batch independence + oracle parity on picked samples
    kw = bench.block_kwargs(model)
    fwd = orc.gated_forward if model.cssm_type == "gated" else orc.gdn_forward
    ref = fwd(variables["params"], x[PICK].cpu().numpy(), **kw)
    assert orc.rel_l2(y[PICK].cpu().numpy(), ref) <= TOL
    # determinism
    y_again = bound(x)
    assert torch.equal(y, y_again)
    # last-frame-only entry point
    y_last = bound(x, last_frame_only=True)
    assert orc.rel_l2(y_last[PICK].cpu().numpy(), ref[:, -1]) <= TOL
    assert torch.allclose(y_last, y[:, -1], rtol=0, atol=1e-5 * float(y[:, -1].abs().max()))
    # causality: change the second half of every clip
    t0 = T // 2
    x2 = x.clone()
    x2[:, t0:] += 0.5
    del y_again, y_last
    y2 = bound(x2)
    assert torch.equal(y2[:, :t0], y[:, :t0])
    assert not torch.equal(y2[:, t0:], y[:, t0:])


@pytest.mark.parametrize("workload", ["cfg2", "cfg3", "cfg4", "gated32", "cfg1"])
def test_model_at_full_size(workload):
    """The bench's own model, weights and synthetic inputs: logits of picked samples against the
    oracle model, logits through the last-frame-only path and through the host-buffer call.
    (cfg1 is the batch-8 configuration: all of its samples are compared.)"""
    model = bench.make_model(workload)
    B = bench.WORKLOADS[workload]["B"]
    PICK = [0, 77, 127] if B == 128 else list(range(B))
    x_np = bench.make_inputs(workload, B, seed0=1000)
    variables = model.init(0, x_np.shape)
    bound = model.bind(variables)
    x = torch.from_numpy(np.ascontiguousarray(x_np)).cuda()
    logits = bound(x)
    assert torch.isfinite(logits).all()
    ref = so.simple_forward(variables["params"], x_np[PICK], cssm_type=model.cssm_type,
                            seq_len=model.seq_len, stem_mode=model.stem_mode,
                            stem_layers=model.stem_layers, pool_type=model.pool_type,
                            readout_norm=model.readout_norm, block_kwargs=bench.block_kwargs(model))
    assert orc.rel_l2(logits[PICK].cpu().numpy(), ref) <= TOL
    last = bound(x, last_frame_only=True)
    assert orc.rel_l2(last.cpu().numpy(), logits.cpu().numpy()) <= 1e-5
    assert torch.equal(bound(x), logits)
    host = bound.forward_host(torch.from_numpy(np.ascontiguousarray(x_np)).pin_memory())
    assert np.array_equal(host.numpy(), logits.cpu().numpy())
