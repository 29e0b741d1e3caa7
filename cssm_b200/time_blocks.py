"""CUDA-event timing of one forward of each block mirror at a given shape:

    python -m cssm_b200.time_blocks --shape 128 8 64 64 64 --blocks additive1 deltanet

Random-init weights and N(0,1) inputs on cuda:0; prints milliseconds per forward (mean of
--steps calls after --warmup).  The model-level benchmark with its JSON contract is bench.py at
the repository root; this is the quick per-block figure.
"""
from __future__ import annotations

import argparse

import torch

from . import AdditiveCSSM, DeltaNetCSSM, GatedCSSM, GatedDeltaNetCSSM, NoGateCSSM


def make(block: str, C: int, ks: int):
    if block == "gated":
        return GatedCSSM(channels=C, kernel_size=ks, gate_type="factored", rope_mode="spatiotemporal")
    if block == "gdn":
        return GatedDeltaNetCSSM(channels=C, kernel_size=ks, delta_key_dim=4, gate_type="factored",
                                 rope_mode="spatiotemporal")
    if block == "nogate":
        return NoGateCSSM(channels=C, kernel_size=ks)
    if block == "additive1":
        return AdditiveCSSM(channels=C, kernel_size=ks, single_state=True, gate_type="factored",
                            rope_mode="spatiotemporal")
    if block == "deltanet":
        return DeltaNetCSSM(channels=C, kernel_size=ks, gate_type="channel", rope_mode="spatiotemporal")
    raise SystemExit(f"unknown block {block!r}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=int, nargs=5, default=[128, 8, 64, 64, 64], metavar=("B", "T", "H", "W", "C"))
    ap.add_argument("--blocks", nargs="+", default=["gated", "gdn", "nogate", "additive1", "deltanet"])
    ap.add_argument("--kernel-size", type=int, default=11)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    B, T, H, W, C = args.shape
    x = torch.randn(B, T, H, W, C, device="cuda")
    y = torch.empty_like(x)
    for name in args.blocks:
        mod = make(name, C, args.kernel_size)
        bound = mod.bind(mod.init(0, tuple(x.shape), bias_scale=0.1))
        for _ in range(args.warmup):
            bound(x, out=y)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            bound(x, out=y)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        print(f"{name:10s} B={B} T={T} {H}x{W} C={C}: {ms:.3f} ms per forward, "
              f"{B / (ms / 1e3):.0f} clips/s", flush=True)


if __name__ == "__main__":
    main()
