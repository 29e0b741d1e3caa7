"""Benchmark of the gated spectral block forward (the hot path) on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload cfg2]

One step = one GatedCSSM block forward over one per-GPU batch of synthetic block inputs.
Prints ONE JSON line (rank 0).  `value` is device-resident throughput; `e2e` goes through
the host-buffer C-ABI entry point with pinned host memory; `roofline` is the fused
spectral kernel timed with CUDA events on its launch stream; `cpu_baseline` is the CPU
restatement of the reference block on the host cores (JAX is not installable here).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE.json configs[1]: Mamba-SCSSM gated, ks 11, factored gates, T=8, C=64, one stem
    # layer (128x128 image -> 64x64 block input), per-GPU batch 128.
    "cfg2": dict(B=128, T=8, H=64, W=64, C=64, kernel_size=11, gate_type="factored",
                 rope_mode="spatiotemporal", short_conv_size=4, short_conv_spatial_size=3),
    # small case for profiler captures (activations 134 MB > L2, < 1 GB on the device)
    "cfg2_small": dict(B=16, T=8, H=64, W=64, C=64, kernel_size=11, gate_type="factored",
                       rope_mode="spatiotemporal", short_conv_size=4, short_conv_spatial_size=3),
    # BASELINE.json configs[0] (main.py defaults: dense gates, 2 stem layers -> 32x32), batch 8
    "cfg1": dict(B=8, T=1, H=32, W=32, C=64, kernel_size=1, gate_type="dense",
                 rope_mode="spatiotemporal", short_conv_size=4, short_conv_spatial_size=3),
    # 32x32 planes at a bandwidth-relevant size (the gated block on the block-input shape of cfg 4)
    "gated32": dict(B=128, T=32, H=32, W=32, C=64, kernel_size=11, gate_type="factored",
                    rope_mode="spatiotemporal", short_conv_size=4, short_conv_spatial_size=3),
    # BASELINE.json configs[2]: GDN-SCSSM, ks 11, qkv_conv 5, d_k 4, T=8, C=64, RMSNorm, mrope
    "cfg3": dict(block="gdn", B=128, T=8, H=64, W=64, C=64, kernel_size=11, gate_type="factored",
                 rope_mode="mrope", short_conv_size=4, qkv_conv_size=5, delta_key_dim=4),
    "cfg3_small": dict(block="gdn", B=8, T=8, H=64, W=64, C=64, kernel_size=11,
                       gate_type="factored", rope_mode="mrope", short_conv_size=4, qkv_conv_size=5,
                       delta_key_dim=4),
    # BASELINE.json configs[3]: GDN-SCSSM video, T=32, 32x32 block input, qkv_conv 1
    "cfg4": dict(block="gdn", B=128, T=32, H=32, W=32, C=64, kernel_size=11, gate_type="factored",
                 rope_mode="spatiotemporal", short_conv_size=4, qkv_conv_size=1, delta_key_dim=4),
}
METRIC = "fwd images/s (gated spectral block, cfg2)"
GDN_STAGES = ["dwconv_ctx", "qkv_proj", "gate_proj", "gates", "short_convs", "spectral", "out_proj"]


def time_last_frame(bound, x, steps, warmup, dev, world):
    """Secondary figure: the same block through the last-frame-only entry point (what a model
    with a last-frame readout consumes).  Returns ms per step, max over ranks."""
    import torch
    from cssm_b200 import shard
    B, T, H, W, Cc = x.shape
    out = torch.empty((B, H, W, Cc), dtype=x.dtype, device=dev)
    for _ in range(max(1, warmup)):
        bound(x, out=out, last_frame_only=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(steps):
        bound(x, out=out, last_frame_only=True)
    e1.record()
    torch.cuda.synchronize(dev)
    return shard.max_over_ranks(e0.elapsed_time(e1), dev) / steps


def run_gdn(args, cfg, rank, world, local):
    """GDN block workloads (not the headline metric): whole-block throughput, per-stage CUDA-event
    times through the library's stage-event hook, roofline of the fused GDN spectral kernel
    (20*C*H*W algorithmic bytes per (b,t): read q,k,v and gate, write o)."""
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist
    from cssm_b200 import GatedDeltaNetCSSM, shard

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, T, H, W, Cc = cfg["B"], cfg["T"], cfg["H"], cfg["W"], cfg["C"]
    mod = GatedDeltaNetCSSM(channels=Cc, delta_key_dim=cfg["delta_key_dim"],
                            kernel_size=cfg["kernel_size"], rope_mode=cfg["rope_mode"],
                            gate_type=cfg["gate_type"], short_conv_size=cfg["short_conv_size"],
                            qkv_conv_size=cfg["qkv_conv_size"])
    bound = mod.bind(mod.init(0, (B, T, H, W, Cc)), dev)
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    x = torch.randn(B, T, H, W, Cc, generator=g).to(dev)
    y = torch.empty_like(x)
    st = torch.cuda.current_stream(dev)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(8)]
    for _ in range(args.warmup):
        bound(x, out=y)
    torch.cuda.synchronize(dev)
    # stage events: raw cudaEvent_t handles of torch events (created on first record)
    for e in evs:
        e.record(st)
    torch.cuda.synchronize(dev)
    arr = (C.c_void_p * 8)(*[e.cuda_event for e in evs])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stage_ms = {n: 0.0 for n in GDN_STAGES}
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    with ClockSampler(local) as clk:
        e0.record(st)
        for k in range(args.steps):
            if k == args.steps - 1:
                bound.L.cssm_debug_gdn_stage_events(arr)
            bound(x, out=y)
        bound.L.cssm_debug_gdn_stage_events(None)
        e1.record(st)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
    for i, n in enumerate(GDN_STAGES):
        stage_ms[n] = evs[i].elapsed_time(evs[i + 1])
    total_ms = shard.max_over_ranks(e0.elapsed_time(e1), dev)
    last_ms = time_last_frame(bound, x, args.steps, args.warmup, dev, world)
    peak, peak_src = peaks()
    alg = 20.0 * Cc * H * W * B * T
    ach = alg / (stage_ms["spectral"] / 1e3) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": f"fwd images/s (GDN spectral block, {args.workload})",
            "value": world * B * args.steps / (total_ms / 1e3), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "block": "GatedDeltaNetCSSM", "per_gpu_batch": B,
                       "T": T, "H": H, "W": W, "C": Cc, "delta_key_dim": cfg["delta_key_dim"],
                       "l2": "inputs larger than the 126 MB L2"},
            "stage_ms": stage_ms,
            "roofline": {"bound": "hbm", "kernel": "gdn_spectral", "achieved": ach, "peak": peak,
                         "peak_source": peak_src, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "algorithmic_bytes_per_launch": alg, "ms_per_launch": stage_ms["spectral"]},
            "last_frame_only": {"ms_per_step": last_ms, "value": world * B / (last_ms / 1e3),
                                "unit": "images/s"},
            "cpu_baseline": None, "e2e": None, "gpu_launches": 9 * args.steps,
            "clocks": clk.summary(),
        }))
    if world > 1:
        dist.destroy_process_group()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs (NVML, read-only)."""
    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
               "sw_power_cap": 0x4}

    def __init__(self, index):
        self.index, self.samples, self.stop = index, [], threading.Event()
        self.th = threading.Thread(target=self.run, daemon=True)
        self.max_mhz = None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            while not self.stop.is_set():
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                     int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
                self.stop.wait(0.005)
        except Exception:
            self._run_smi()

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v for v in vis.split(",") if v.strip() != ""]
            if self.index < len(ids) and ids[self.index].strip().isdigit():
                return int(ids[self.index])
        return self.index

    def _run_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self._physical_index()),
                                      f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                f = [x.strip() for x in out.split(",")]
                if len(f) >= 6:
                    self.max_mhz = float(f[1])
                    mask = sum(self.REASONS[n] for i, n in enumerate(names)
                               if f[2 + i].lower().startswith("active"))
                    self.samples.append((float(f[0]), mask))
            except Exception:
                pass
            self.stop.wait(0.05)

    def __enter__(self):
        self.th.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.th.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        sm = sorted(s[0] for s in self.samples)
        reasons = [n for n, bit in self.REASONS.items() if any(s[1] & bit for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_rate(cfg, sample_b, reps=1):
    """images/s of the CPU restatement (torch-CPU, all host threads) on `sample_b` images of
    the workload."""
    import numpy as np
    import torch
    from oracle import cssm_oracle as orc
    from oracle import cssm_torch_cpu as tc
    p = orc.init_gated_params(1, cfg["C"], cfg["H"], cfg["W"], kernel_size=cfg["kernel_size"],
                              gate_type=cfg["gate_type"], short_conv_size=cfg["short_conv_size"],
                              short_conv_spatial_size=cfg["short_conv_spatial_size"])
    g = torch.Generator().manual_seed(0)
    x = torch.randn(sample_b, cfg["T"], cfg["H"], cfg["W"], cfg["C"], generator=g)
    kw = dict(kernel_size=cfg["kernel_size"], rope_mode=cfg["rope_mode"], gate_type=cfg["gate_type"],
              short_conv_size=cfg["short_conv_size"],
              short_conv_spatial_size=cfg["short_conv_spatial_size"])
    tc.gated_forward_torch(p, x[:1], **kw)           # touch code paths once
    t0 = time.perf_counter()
    for _ in range(reps):
        tc.gated_forward_torch(p, x, **kw)
    dt = (time.perf_counter() - t0) / reps
    return sample_b / dt, dt, torch.get_num_threads()


def run_reference(args, cfg, rank):
    if rank != 0:
        return
    sample_b = 16
    times = []
    for i in range(args.warmup + args.steps):
        rate, dt, cores = cpu_reference_rate(cfg, sample_b)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = sample_b / (ms / 1e3)
    sample = (f"{sample_b} images of the {args.workload} block input per step "
              f"(T={cfg['T']}, {cfg['H']}x{cfg['W']}, C={cfg['C']}), torch-CPU restatement")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": args.workload, "sample_batch": sample_b},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-chunk", type=int, default=8, help="images per host<->device chunk")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from cssm_b200 import GatedCSSM, synth
    from cssm_b200._lib import check

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: cssm_b200 has no CPU path")
    if cfg.get("block") == "gdn":
        run_gdn(args, cfg, rank, world, local)
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, T, H, W, Cc = cfg["B"], cfg["T"], cfg["H"], cfg["W"], cfg["C"]
    mod = GatedCSSM(channels=Cc, kernel_size=cfg["kernel_size"], rope_mode=cfg["rope_mode"],
                    gate_type=cfg["gate_type"], short_conv_size=cfg["short_conv_size"],
                    short_conv_spatial_size=cfg["short_conv_spatial_size"])
    variables = mod.init(0, (B, T, H, W, Cc))
    bound = mod.bind(variables, dev)

    # synthetic block input: stem features of seeded stroke images (16 distinct images per
    # rank, tiled to the batch), disjoint seeds per rank
    stem_layers = {64: 1, 32: 2}[H]          # 128x128 stroke images, one 2x pool per stem layer
    base = synth.stem_features(synth.stroke_batch(16, seed0=1000 + 16 * rank), T, Cc,
                               layers=stem_layers)
    assert base.shape[2:4] == (H, W)
    x_host = torch.from_numpy(np.tile(base, (B // 16 + 1, 1, 1, 1, 1))[:B]).contiguous()
    x = x_host.to(dev)
    y = torch.empty_like(x)

    d = bound.desc(tuple(x.shape))
    pl = bound.plan(d)
    lay = bound.workspace_layout(d)
    ws = torch.empty(lay.total, dtype=torch.uint8, device=dev)
    L = bound.L
    st = torch.cuda.current_stream(dev)
    sp = st.cuda_stream
    wsb = ws.data_ptr()
    stage_names = ["in_proj", "short_conv", "gates", "spectral", "out_proj"]

    def step(evs=None):
        calls = [
            lambda: L.cssm_gated_in_proj(C.byref(d), C.byref(bound.w), pl.data_ptr(), x.data_ptr(),
                                         wsb + lay.xz_planar, sp),
            lambda: L.cssm_gated_short_conv(C.byref(d), C.byref(bound.w), wsb + lay.xz_planar,
                                            wsb + lay.ctx_sum, sp),
            lambda: L.cssm_gated_gates(C.byref(d), C.byref(bound.w), wsb + lay.ctx_sum,
                                       wsb + lay.gate_maps, sp),
            lambda: L.cssm_gated_spectral(C.byref(d), pl.data_ptr(), wsb + lay.gate_maps,
                                          wsb + lay.xz_planar, sp),
            lambda: L.cssm_gated_out_proj(C.byref(d), C.byref(bound.w), wsb + lay.xz_planar,
                                          y.data_ptr(), sp),
        ]
        for i, c in enumerate(calls):
            if evs is not None:
                evs[i][0].record(st)
            check(c(), stage_names[i])
            if evs is not None:
                evs[i][1].record(st)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            for _ in stage_names] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    clk = ClockSampler(local)
    clk.__enter__()                       # sampled over the device-timed and the e2e regions
    e0.record(st)
    for k in range(args.steps):
        step(evs[k])
    e1.record(st)
    barrier()
    total_ms = e0.elapsed_time(e1)
    if world > 1:
        tt = torch.tensor([total_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    ms_step = total_ms / args.steps
    value = world * B * args.steps / (total_ms / 1e3)
    stage_ms = {n: sum(evs[k][i][0].elapsed_time(evs[k][i][1]) for k in range(args.steps)) / args.steps
                for i, n in enumerate(stage_names)}

    # roofline of the fused spectral kernel: 12*H*W bytes per (b,t,c) plane-step
    peak, peak_src = peaks()
    alg_bytes = 12.0 * H * W * B * T * Cc
    achieved = alg_bytes / (stage_ms["spectral"] / 1e3) / 1e9
    roofline = {"bound": "hbm", "kernel": "gated_spectral_r64" if H == 64 else "gated_spectral_r32", "achieved": achieved, "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8TBps": achieved / 8000.0, "traffic": None,
                "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": stage_ms["spectral"]}
    tr = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tr):
        with open(tr) as f:
            per_plane_step = json.load(f).get("gated_spectral_r64_dram_bytes_per_plane_step")
        if per_plane_step:
            roofline["traffic"] = per_plane_step * B * T * Cc

    last_ms = time_last_frame(bound, x, args.steps, args.warmup, dev, world)

    # end to end through the host-buffer entry point (pinned host memory)
    e2e = None
    if not args.no_e2e:
        chunk = min(args.e2e_chunk, B)
        xh = x_host.pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        n = L.cssm_gated_host_workspace_bytes(C.byref(d), chunk)
        hws = torch.empty(n, dtype=torch.uint8, device=dev)

        def host_step():
            check(L.cssm_gated_forward_host(C.byref(d), C.byref(bound.w), pl.data_ptr(),
                                            xh.data_ptr(), yh.data_ptr(), chunk, hws.data_ptr(), n, sp),
                  "forward_host")
        for _ in range(max(1, min(args.warmup, 3))):
            host_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            host_step()
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        if world > 1:
            tt = torch.tensor([dt], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
        nbytes = x.numel() * 4
        e2e = {"value": world * B * args.steps / dt, "unit": "images/s",
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
               "ms_per_step": 1e3 * dt / args.steps, "chunk_batch": chunk}
        del hws, xh, yh
    clk.__exit__(None, None, None)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        rate, dt, cores = cpu_reference_rate(cfg, 16, reps=16)
        cpu = {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
               "sample": f"16 images of the {args.workload} block input, 16 repetitions "
                         f"({dt:.2f} s each), torch-CPU restatement of the reference block"}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "block": "GatedCSSM", "per_gpu_batch": B, "T": T,
                       "H": H, "W": W, "C": Cc, "kernel_size": cfg["kernel_size"],
                       "gate_type": cfg["gate_type"], "rope_mode": cfg["rope_mode"],
                       "l2": "inputs (1.07 GB per tensor at cfg2) larger than the 126 MB L2"},
            "stage_ms": stage_ms, "roofline": roofline,
            "last_frame_only": {"ms_per_step": last_ms, "value": world * B / (last_ms / 1e3),
                                "unit": "images/s"},
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": 5 * args.steps, "clocks": clk.summary(),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
