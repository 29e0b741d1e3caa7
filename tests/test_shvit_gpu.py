"""GPU tests of the bf16 kernels under the CSSM-SHViT model, through the C ABI: the tcgen05 GEMM
with its K loop and epilogue options, the 3x3 stride-2 convolution as an implicit GEMM (both
against float32 torch references on the same bf16-rounded operands), the model's intermediate
activations against the NumPy oracle, and run-to-run determinism.  Tolerance 2e-2 (bf16)."""
import ctypes as C

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from cssm_b200 import CSSMSHViT, device_error, lib
from cssm_b200._lib import check
from oracle import cssm_oracle as orc
from oracle import shvit_oracle as sv

pytestmark = pytest.mark.gpu


def _st():
    return torch.cuda.current_stream().cuda_stream


def _pack(L, kernel, K, N, col_scale=None):
    ld = L.cssm_bf16_packed_ld(K)
    wt = torch.empty((N, ld), dtype=torch.bfloat16, device="cuda")
    cs = col_scale.data_ptr() if col_scale is not None else None
    check(L.cssm_bf16_pack_weight(kernel.data_ptr(), K, N, cs, wt.data_ptr(), _st()), "pack")
    return wt


@pytest.mark.parametrize("M,K,N,act,res", [
    (300, 64, 64, 0, False), (1000, 256, 512, 1, False), (777, 1024, 256, 0, True),
    (128, 384, 1536, 1, False), (5000, 1536, 384, 0, True), (1, 64, 128, 2, False),
    (20000, 128, 128, 2, True), (257, 512, 768, 2, False), (129, 64, 1024, 0, False)])
def test_bf16_gemm(M, K, N, act, res):
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    A = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
    W = (torch.randn((K, N), device="cuda", generator=g) / K ** 0.5)
    b = torch.randn((N,), device="cuda", generator=g)
    R = torch.randn((M, N), device="cuda", generator=g).to(torch.bfloat16) if res else None
    wt = _pack(L, W, K, N)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    check(L.cssm_bf16_gemm(A.data_ptr(), M, K, wt.data_ptr(), N, b.data_ptr(), act,
                           R.data_ptr() if res else None, out.data_ptr(), _st()), "gemm")
    ref = A.float() @ W.to(torch.bfloat16).float() + b
    if act == 1:
        ref = F.gelu(ref, approximate="tanh")
    elif act == 2:
        ref = F.silu(ref)
    if res:
        ref = ref + R.float()
    torch.cuda.synchronize()
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 6e-3, float(err)          # one bf16 rounding of the output


@pytest.mark.parametrize("B,Hi,Wi,Cin,Cout", [(2, 16, 16, 32, 64), (3, 14, 14, 128, 256),
                                              (2, 7, 9, 64, 128), (1, 56, 56, 64, 128),
                                              (2, 112, 112, 32, 64), (5, 14, 14, 256, 384),
                                              (2, 9, 7, 32, 64), (3, 28, 28, 128, 256), (2, 12, 20, 16, 32),
                                              (1, 300, 260, 64, 64)])
def test_bf16_conv3x3s2(B, Hi, Wi, Cin, Cout):
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(Hi * Cin)
    x = torch.randn((B, Hi, Wi, Cin), device="cuda", generator=g).to(torch.bfloat16)
    W = torch.randn((3, 3, Cin, Cout), device="cuda", generator=g) / (9 * Cin) ** 0.5
    scale = 1.0 + 0.2 * torch.randn((Cout,), device="cuda", generator=g)
    b = torch.randn((Cout,), device="cuda", generator=g)
    wt = torch.empty((Cout, L.cssm_bf16_conv3x3s2_packed_ld(Cin, Wi, Cout)), dtype=torch.bfloat16, device="cuda")
    check(L.cssm_bf16_pack_conv3x3s2_weight(W.data_ptr(), Cin, Cout, Wi, scale.data_ptr(), wt.data_ptr(), _st()),
          "pack_conv")
    Ho, Wo = (Hi + 1) // 2, (Wi + 1) // 2
    out = torch.empty((B, Ho, Wo, Cout), dtype=torch.bfloat16, device="cuda")
    check(L.cssm_bf16_conv3x3s2(x.data_ptr(), B, Hi, Wi, Cin, wt.data_ptr(), Cout, b.data_ptr(), 0,
                                out.data_ptr(), _st()), "conv")
    th, tw = max((Ho - 1) * 2 + 3 - Hi, 0), max((Wo - 1) * 2 + 3 - Wi, 0)
    xp = F.pad(x.float().permute(0, 3, 1, 2), (tw // 2, tw - tw // 2, th // 2, th - th // 2))
    wq = (W * scale).to(torch.bfloat16).float().permute(3, 2, 0, 1)
    ref = F.conv2d(xp, wq, b, stride=2).permute(0, 2, 3, 1)
    torch.cuda.synchronize()
    assert out.shape == ref.shape
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 6e-3, float(err)


@pytest.mark.parametrize("M", [1, 300, 128 * 148 + 64, 128 * 148 * 5 + 17])
def test_bf16_fused_mlp(M):
    """fc1 -> gelu -> fc2 -> + residual in one kernel (C = 64, Hd = 256) against float32 torch on the same
    bf16 operands, with the hidden layer rounded to bf16 as the kernel and the two-GEMM path round it;
    ragged last tiles, fewer tiles than CTAs, several tiles per CTA."""
    L = lib()
    Cd, Hd = 64, 256
    g = torch.Generator(device="cuda").manual_seed(M)
    A = torch.randn((M, Cd), device="cuda", generator=g).to(torch.bfloat16)
    R = torch.randn((M, Cd), device="cuda", generator=g).to(torch.bfloat16)
    W1 = torch.randn((Cd, Hd), device="cuda", generator=g) / Cd ** 0.5
    W2 = torch.randn((Hd, Cd), device="cuda", generator=g) / Hd ** 0.5
    b1 = torch.randn((Hd,), device="cuda", generator=g)
    b2 = torch.randn((Cd,), device="cuda", generator=g)
    w1t, w2t = _pack(L, W1, Cd, Hd), _pack(L, W2, Hd, Cd)
    out = torch.full((M, Cd), float("nan"), dtype=torch.bfloat16, device="cuda")
    check(L.cssm_bf16_mlp(A.data_ptr(), M, Cd, Hd, w1t.data_ptr(), b1.data_ptr(), w2t.data_ptr(),
                          b2.data_ptr(), R.data_ptr(), out.data_ptr(), _st()), "mlp")
    hid = F.gelu(A.float() @ W1.to(torch.bfloat16).float() + b1, approximate="tanh").to(torch.bfloat16)
    ref = hid.float() @ W2.to(torch.bfloat16).float() + b2 + R.float()
    torch.cuda.synchronize()
    assert device_error() == 0
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 6e-3, float(err)
    # the same through the two GEMM calls the model uses for every other size
    h2 = torch.empty((M, Hd), dtype=torch.bfloat16, device="cuda")
    o2 = torch.empty((M, Cd), dtype=torch.bfloat16, device="cuda")
    check(L.cssm_bf16_gemm(A.data_ptr(), M, Cd, w1t.data_ptr(), Hd, b1.data_ptr(), 1, None, h2.data_ptr(), _st()), "fc1")
    check(L.cssm_bf16_gemm(h2.data_ptr(), M, Hd, w2t.data_ptr(), Cd, b2.data_ptr(), 0, R.data_ptr(), o2.data_ptr(), _st()), "fc2")
    torch.cuda.synchronize()
    assert (out.float() - o2.float()).norm() / o2.float().norm() < 6e-3
    assert L.cssm_bf16_mlp(A.data_ptr(), M, 128, 512, w1t.data_ptr(), b1.data_ptr(), w2t.data_ptr(),
                           b2.data_ptr(), R.data_ptr(), out.data_ptr(), _st()) != 0


_TINY = dict(embed_dims=(32, 64, 64, 128), depths=(1, 1, 2, 1), num_classes=10, num_timesteps=1,
             kernel_sizes=(1, 1, 1, 1), short_conv_spatial_size=0)


def test_model_fast_path_matches_oracle_and_is_deterministic():
    """A small CSSM-SHViT whose CSSM stages have 14x14 and 7x7 planes (224-pixel input), so the
    bf16 channels-last mixer path runs; logits against the fp64 oracle, twice, bit-identical."""
    p, s = sv.init_shvit_params(7, (224, 224), **{k: v for k, v in _TINY.items() if k != "num_timesteps"})
    x = np.random.default_rng(3).standard_normal((3, 224, 224, 3)).astype(np.float32)
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    ref = sv.shvit_forward(p, s, xb.float().cpu().numpy().astype(np.float64),
                           **{k: v for k, v in _TINY.items() if k != "num_classes"})
    model = CSSMSHViT(**_TINY)
    variables = {"params": p, "batch_stats": s}
    y1 = model.apply(variables, xb).clone()
    y2 = model.apply(variables, xb)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert orc.rel_l2(y1.cpu().numpy(), ref) <= 2e-2


def test_host_entry_matches_device_entry():
    p, s = sv.init_shvit_params(8, (64, 64), embed_dims=(32, 32, 64, 64), depths=(1, 1, 1, 1), num_classes=7,
                                kernel_sizes=(3, 3, 3, 3))
    model = CSSMSHViT(embed_dims=(32, 32, 64, 64), depths=(1, 1, 1, 1), num_classes=7, num_timesteps=2,
                      kernel_sizes=(3, 3, 3, 3))
    bound = model.bind({"params": p, "batch_stats": s})
    x = torch.randn((2, 64, 64, 3)).to(torch.bfloat16)
    want = bound(x.cuda()).cpu()
    xh, lh = x.pin_memory(), torch.empty((2, 7), dtype=torch.float32).pin_memory()
    bound.forward_host(xh, lh)
    assert torch.equal(lh, want)
    # a batch that the host entry point cuts into two overlapped chunks
    x = torch.randn((64, 64, 64, 3)).to(torch.bfloat16)
    want = bound(x.cuda()).cpu()
    xh, lh = x.pin_memory(), torch.empty((64, 7), dtype=torch.float32).pin_memory()
    bound.forward_host(xh, lh)
    assert torch.equal(lh, want)
    # the launch trace covers the whole forward and changes nothing
    logits, launches = bound.forward_traced(x.cuda())
    assert torch.equal(logits.cpu(), want)
    kinds = [k for k, _, _ in launches]
    assert kinds[0] == "stem_conv" and kinds[-1] == "head" and "gemm" in kinds and "conv_gemm" in kinds
    assert all(ms >= 0 for _, ms, _ in launches)


def test_streaming_host_entry_prefetches_the_next_batch():
    """forward_host_pipelined: a batch that the previous call prefetched, a batch that nobody
    prefetched, and a prefetch that is never used all give the device entry point's logits."""
    p, s = sv.init_shvit_params(9, (64, 64), embed_dims=(32, 32, 64, 64), depths=(1, 1, 1, 1), num_classes=7,
                                kernel_sizes=(3, 3, 3, 3))
    model = CSSMSHViT(embed_dims=(32, 32, 64, 64), depths=(1, 1, 1, 1), num_classes=7, num_timesteps=2,
                      kernel_sizes=(3, 3, 3, 3))
    bound = model.bind({"params": p, "batch_stats": s})
    xs = [torch.randn((16, 64, 64, 3)).to(torch.bfloat16).pin_memory() for _ in range(4)]
    want = [bound(x.cuda()).cpu() for x in xs]
    lh = torch.empty((16, 7), dtype=torch.float32).pin_memory()
    bound.forward_host_pipelined(xs[0], xs[1], lh)          # cold: copies xs[0] itself, prefetches xs[1]
    assert torch.equal(lh, want[0])
    bound.forward_host_pipelined(xs[1], xs[2], lh)          # prefetched
    assert torch.equal(lh, want[1])
    bound.forward_host_pipelined(xs[3], None, lh)           # the prefetch of xs[2] is dropped
    assert torch.equal(lh, want[3])
    bound.forward_host_pipelined(xs[2], xs[2], lh)          # nothing prefetched; next = the same buffer
    assert torch.equal(lh, want[2])
    bound.forward_host_pipelined(xs[2], None, lh)
    assert torch.equal(lh, want[2])
    bound.close()
    bound.forward_host_pipelined(xs[0], None, lh)           # a new pipe after close()
    assert torch.equal(lh, want[0])
    bound.close()


def test_cfg5_full_batch_picked_samples():
    """BASELINE configs[4] at its full size (cssm_shvit_s1, T = 1, kernel_size 1, batch 512 of
    224x224x3 bf16 N(0,1) images, 1000 classes): logits of samples picked out of the batch against the
    fp64 oracle run on those samples alone (samples are independent), 2e-2."""
    import bench
    p, s = bench.shvit_params("cfg5")
    model = CSSMSHViT(**bench.WORKLOADS["cfg5"]["model"])
    bound = model.bind({"params": p, "batch_stats": s})
    x = torch.from_numpy(bench.make_inputs("cfg5", 512, seed0=77)).to(torch.bfloat16)
    y = bound(x.cuda()).cpu().numpy()
    assert np.isfinite(y).all() and y.shape == (512, 1000)
    pick = [0, 255, 511]
    ref = sv.shvit_forward(p, s, x[pick].float().numpy().astype(np.float64), **bench.shvit_model_kwargs("cfg5"))
    for i, b in enumerate(pick):
        assert orc.rel_l2(y[b], ref[i]) <= 2e-2, (b, orc.rel_l2(y[b], ref[i]))
