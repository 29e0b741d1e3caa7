"""Benchmark of the CSSM spectral-block forward on B200: model-level images/s, per-kernel / per-stage
CUDA-event times, roofline of the dominant kernel, end-to-end figure through the host-buffer entry
points, CPU restatement beside it.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

One step = one forward of the workload's model over one per-GPU batch of seeded synthetic inputs.
Without --workload the headline is cfg5 (BASELINE.json configs[4], the configuration the metric
"fwd images/s at 1/2/4/8 B200" names: CSSM-SHViT s1, gated mixers at T = 1, bf16, batch 512 per GPU)
and the SimpleCSSM workloads cfg1 .. cfg4 (configs[0..3], fp32) run after it and are reported
under "workloads" in the same JSON line (rank 0 prints ONE line):
  value     images/s, inputs resident on the device, CUDA events around the K timed steps
  e2e       the same through the host-buffer entry point: pinned host inputs in, host logits out
  roofline  the dominant kernel: algorithmic bytes / its CUDA-event time, vs the measured HBM peak
  kernels / block / stage_ms   per-kernel (cfg5: launch trace) or per-stage (SimpleCSSM) event times
  sustained the headline loop repeated for >= 2 s, with the median SM clock seen
  cpu_baseline   the CPU restatement of the same model on the host cores (JAX cannot be installed
                 here, so the reference itself cannot run)
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

_GATED = dict(cssm_type="gated", embed_dim=64, num_classes=2, short_conv_size=4, short_conv_spatial_size=3)
_GDN = dict(cssm_type="gdn", embed_dim=64, num_classes=2, short_conv_size=4, delta_key_dim=4,
            gate_type="factored", output_norm="rms")
WORKLOADS = {
    # BASELINE.json configs[1]: Mamba-SCSSM gated, ks 11, factored gates, T=8 (image repeated),
    # embed_dim 64, depth 1, one stem layer (128x128 -> 64x64), max-pool + linear 2-way head
    "cfg2": dict(model=dict(_GATED, kernel_size=11, gate_type="factored", seq_len=8, stem_layers=1,
                            pool_type="max", pos_embed="spatiotemporal"),
                 B=128, data="strokes"),
    # the same model at a size for profiler captures (activations 134 MB > L2, < 1 GB on the device)
    "cfg2_small": dict(model=dict(_GATED, kernel_size=11, gate_type="factored", seq_len=8, stem_layers=1,
                                  pool_type="max", pos_embed="spatiotemporal"),
                       B=16, data="strokes"),
    # BASELINE.json configs[0] (main.py defaults: dense gates, two stem layers -> 32x32, mean pool)
    "cfg1": dict(model=dict(_GATED, kernel_size=1, gate_type="dense", seq_len=1, stem_layers=2,
                            pool_type="mean", pos_embed="spatiotemporal"),
                 B=8, data="strokes"),
    # 32x32 planes at a bandwidth-relevant size: the gated model on the clip input of configs[3]
    "gated32": dict(model=dict(_GATED, kernel_size=11, gate_type="factored", stem_mode="pathtracker",
                               pool_type="max", pos_embed="spatiotemporal"),
                    B=128, data="dots"),
    # BASELINE.json configs[2]: GDN-SCSSM, ks 11, qkv_conv 5, d_k 4, T=8, RMSNorm, mrope
    "cfg3": dict(model=dict(_GDN, kernel_size=11, qkv_conv_size=5, seq_len=8, stem_layers=1,
                            pool_type="max", pos_embed="mrope"),
                 B=128, data="strokes"),
    "cfg3_small": dict(model=dict(_GDN, kernel_size=11, qkv_conv_size=5, seq_len=8, stem_layers=1,
                                  pool_type="max", pos_embed="mrope"),
                       B=8, data="strokes"),
    "cfg4_small": dict(model=dict(_GDN, kernel_size=11, qkv_conv_size=1, stem_mode="pathtracker",
                                  pool_type="max", pos_embed="spatiotemporal"),
                       B=8, data="dots"),
    # BASELINE.json configs[3]: GDN-SCSSM video, T=32 native 32x32x3 frames, last-frame readout
    "cfg4": dict(model=dict(_GDN, kernel_size=11, qkv_conv_size=1, stem_mode="pathtracker",
                            pool_type="max", pos_embed="spatiotemporal"),
                 B=128, data="dots"),
}
# BASELINE.json configs[4]: CSSM-SHViT s1, gated mixers at T = 1, kernel_size 1 (no spatial short conv),
# 1000 classes, bf16, batch 512 per GPU of 224x224x3 N(0,1) images
_SHVIT = dict(num_classes=1000, embed_dims=(64, 128, 256, 384), depths=(1, 2, 2, 1), num_timesteps=1,
              kernel_sizes=(1, 1, 1, 1), short_conv_size=4, short_conv_spatial_size=0, gate_type="factored")
WORKLOADS["cfg5"] = dict(kind="shvit", model=_SHVIT, B=512, data="gaussian", hw=224)
# the same model at a size for profiler captures (stage-0 activations 13 MB per tensor... x 32 images)
WORKLOADS["cfg5_small"] = dict(kind="shvit", model=_SHVIT, B=128, data="gaussian", hw=224)
GATED_STAGES = ["in_proj", "short_conv", "gates", "spectral", "out_proj"]
GDN_STAGES = ["dwconv_ctx", "qkv_proj", "gate_proj", "gates", "short_convs", "spectral", "out_proj"]


def is_shvit(workload):
    return WORKLOADS[workload].get("kind") == "shvit"


def metric_name(workload):
    if is_shvit(workload):
        return f"fwd images/s (CSSM-SHViT s1, gated mixers, bf16, {workload})"
    return f"fwd images/s (SimpleCSSM {WORKLOADS[workload]['model']['cssm_type']} model, {workload})"


def make_model(workload):
    from cssm_b200 import SimpleCSSM
    return SimpleCSSM(**WORKLOADS[workload]["model"])


def make_inputs(workload, n, seed0):
    """Seeded synthetic inputs: dashed-stroke images (B,128,128,1), random-walk dot clips
    (B,32,32,32,3) or N(0,1) images (B,224,224,3) (stand-ins for Pathfinder / PathTracker / ImageNet)."""
    from cssm_b200 import synth
    if WORKLOADS[workload]["data"] == "gaussian":
        import numpy as np
        hw = WORKLOADS[workload]["hw"]
        return np.random.default_rng(seed0).standard_normal((n, hw, hw, 3), dtype=np.float32)
    if WORKLOADS[workload]["data"] == "strokes":
        return synth.stroke_batch(n, seed0=seed0)
    return synth.dot_clips(n, seed0=seed0)


def block_kwargs(model):
    """Keyword arguments of the oracle block functions for a SimpleCSSM mirror."""
    rope = model.pos_embed if model.pos_embed in ("spatiotemporal", "spatial_only", "temporal", "mrope") else "none"
    if model.cssm_type == "gated":
        return dict(kernel_size=model.kernel_size, rope_mode=rope, gate_type=model.gate_type,
                    short_conv_size=model.short_conv_size,
                    short_conv_spatial_size=model.short_conv_spatial_size)
    return dict(delta_key_dim=model.delta_key_dim, kernel_size=model.kernel_size, rope_mode=rope,
                gate_type=model.gate_type, short_conv_size=model.short_conv_size,
                qkv_conv_size=model.qkv_conv_size)


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


def shvit_model_kwargs(workload):
    """Keyword arguments of oracle.shvit_oracle / cssm_torch_cpu for a CSSM-SHViT workload."""
    m = WORKLOADS[workload]["model"]
    return {k: m[k] for k in ("embed_dims", "depths", "num_timesteps", "kernel_sizes", "short_conv_size",
                              "short_conv_spatial_size", "gate_type")}


def shvit_params(workload, seed=0):
    from oracle import shvit_oracle as sv
    m, hw = WORKLOADS[workload]["model"], WORKLOADS[workload]["hw"]
    return sv.init_shvit_params(seed, (hw, hw), embed_dims=m["embed_dims"], depths=m["depths"],
                                kernel_sizes=m["kernel_sizes"], num_classes=m["num_classes"],
                                gate_type=m["gate_type"], short_conv_size=m["short_conv_size"],
                                short_conv_spatial_size=m["short_conv_spatial_size"])


def cpu_model_rate(workload, sample_b, reps=1):
    """images/s of the CPU restatement of the workload's model (torch-CPU, all host threads) on
    `sample_b` inputs.  Returns (images/s, seconds per repetition, threads)."""
    import numpy as np
    import torch
    from oracle import simple_oracle as so
    from oracle import cssm_torch_cpu as tc
    # all host threads this process may use (torchrun presets OMP_NUM_THREADS=1 for its workers)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    if is_shvit(workload):
        p, st = shvit_params(workload)
        kw = shvit_model_kwargs(workload)
        xt = torch.from_numpy(make_inputs(workload, sample_b, seed0=3000))
        with torch.no_grad():
            tc.shvit_forward_torch(p, st, xt[:1], **kw)          # touch code paths once
            t0 = time.perf_counter()
            for _ in range(reps):
                tc.shvit_forward_torch(p, st, xt, **kw)
            dt = (time.perf_counter() - t0) / reps
        return sample_b / dt, dt, torch.get_num_threads()
    m = make_model(workload)
    x = make_inputs(workload, sample_b, seed0=3000)
    H, W = m.feature_hw(x.shape[-3], x.shape[-2])
    kw = block_kwargs(m)
    p = so.init_simple_params(1, cin=x.shape[-1], embed_dim=m.embed_dim, H=H, W=W,
                              num_classes=m.num_classes, cssm_type=m.cssm_type,
                              stem_mode=m.stem_mode, stem_layers=m.stem_layers, bias_scale=0.0,
                              block_kwargs=kw)
    xt = torch.from_numpy(np.ascontiguousarray(x))
    run = lambda xx: tc.simple_forward_torch(p, xx, cssm_type=m.cssm_type, seq_len=m.seq_len,
                                             stem_mode=m.stem_mode, stem_layers=m.stem_layers,
                                             pool_type=m.pool_type, readout_norm=m.readout_norm,
                                             block_kwargs=kw)
    with torch.no_grad():
        run(xt[:1])                                  # touch code paths once
        t0 = time.perf_counter()
        for _ in range(reps):
            run(xt)
        dt = (time.perf_counter() - t0) / reps
    return sample_b / dt, dt, torch.get_num_threads()


def cpu_sample_size(workload):
    """Inputs per CPU step, sized so that a step takes seconds, not minutes."""
    if is_shvit(workload):
        return 64
    return 4 if WORKLOADS[workload]["model"]["cssm_type"] == "gdn" else 16


def run_reference(args, rank):
    """Reference arm: the CPU restatement of the same model on the host cores (rank 0 only)."""
    if rank != 0:
        return
    sample_b = min(cpu_sample_size(args.workload), WORKLOADS[args.workload]["B"])
    times = []
    cores = 0
    for i in range(args.warmup + args.steps):
        _, dt, cores = cpu_model_rate(args.workload, sample_b)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = sample_b / (ms / 1e3)
    sample = (f"{sample_b} inputs of the {args.workload} model per step, torch-CPU (float32) restatement "
              f"of the reference model (all T frames computed as the reference does)")
    print(json.dumps({
        "impl": "reference", "metric": metric_name(args.workload), "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if is_shvit(args.workload) else "f32",
        "data": "synthetic", "config": {"workload": args.workload, "sample_batch": sample_b},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def time_region(fn, steps, dev, st):
    """CUDA-event time of `steps` calls of fn on stream st (ms), max over ranks."""
    import torch
    from cssm_b200 import shard
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record(st)
    for _ in range(steps):
        fn()
    e1.record(st)
    torch.cuda.synchronize(dev)
    return shard.max_over_ranks(e0.elapsed_time(e1), dev)


def block_stage_times(bound, feat5, steps, dev, st):
    """Per-stage CUDA-event times (ms, mean over `steps`) of the block alone on its (B,T,H,W,C)
    input.  Gated block: the five stage entry points with an event pair around each; GDN block:
    the library's stage-event hook."""
    import torch
    from cssm_b200._lib import check
    blk = bound.block
    L = blk.L
    if bound.mod.cssm_type == "gated":
        d = blk.desc(tuple(feat5.shape))
        pl = blk.plan(d)
        lay = blk.workspace_layout(d)
        ws = blk.buf.get("ws", lay.total)
        y = torch.empty_like(feat5)
        wsb, sp = ws.data_ptr(), st.cuda_stream
        calls = [
            lambda: L.cssm_gated_in_proj(C.byref(d), C.byref(blk.w), pl.data_ptr(), feat5.data_ptr(),
                                         wsb + lay.xz_planar, sp),
            lambda: L.cssm_gated_short_conv(C.byref(d), C.byref(blk.w), wsb + lay.xz_planar,
                                            wsb + lay.ctx_sum, sp),
            lambda: L.cssm_gated_gates(C.byref(d), C.byref(blk.w), wsb + lay.ctx_sum,
                                       wsb + lay.gate_maps, sp),
            lambda: L.cssm_gated_spectral(C.byref(d), pl.data_ptr(), wsb + lay.gate_maps,
                                          wsb + lay.xz_planar, sp),
            lambda: L.cssm_gated_out_proj(C.byref(d), C.byref(blk.w), wsb + lay.xz_planar,
                                          y.data_ptr(), sp),
        ]
        evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                for _ in GATED_STAGES] for _ in range(steps)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for c in calls:
            check(c(), "stage")                       # warm
        torch.cuda.synchronize(dev)
        e0.record(st)
        for k in range(steps):
            for i, c in enumerate(calls):
                evs[k][i][0].record(st)
                check(c(), GATED_STAGES[i])
                evs[k][i][1].record(st)
        e1.record(st)
        torch.cuda.synchronize(dev)
        stage = {n: sum(evs[k][i][0].elapsed_time(evs[k][i][1]) for k in range(steps)) / steps
                 for i, n in enumerate(GATED_STAGES)}
        return stage, e0.elapsed_time(e1) / steps
    y = torch.empty_like(feat5)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(8)]
    blk(feat5, out=y)
    d = blk.desc(tuple(feat5.shape))
    plan = blk.plan(d)
    ws = blk.buf.get("ws", L.cssm_gdn_workspace_bytes(C.byref(d)))
    for e in evs:
        e.record(st)                                  # creates the raw cudaEvent_t handles
    torch.cuda.synchronize(dev)
    arr = (C.c_void_p * 8)(*[e.cuda_event for e in evs])
    stage = {n: 0.0 for n in GDN_STAGES}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for k in range(steps):
        check(L.cssm_gdn_forward_timed(C.byref(d), C.byref(blk.w), plan.data_ptr(), feat5.data_ptr(),
                                       y.data_ptr(), ws.data_ptr(), ws.numel(), st.cuda_stream, arr),
              "gdn_forward_timed")
        torch.cuda.synchronize(dev)
        for i, n in enumerate(GDN_STAGES):
            stage[n] += evs[i].elapsed_time(evs[i + 1]) / steps
    e1.record(st)
    torch.cuda.synchronize(dev)
    return stage, sum(stage.values())


def run_shvit(args, name, ctx):
    """One CSSM-SHViT workload: device-timed model steps, launch trace (per-kernel times and
    algorithmic bytes), end to end through the host entry point, CPU restatement."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from cssm_b200 import CSSMSHViT, shard
    dev, st, world, rank = ctx["dev"], ctx["st"], ctx["world"], ctx["rank"]
    wl = WORKLOADS[name]
    B = wl["B"]
    model = CSSMSHViT(**wl["model"])
    p, stats = shvit_params(name)
    bound = model.bind({"params": p, "batch_stats": stats}, dev)
    x_host = torch.from_numpy(make_inputs(name, B, seed0=1000 + B * rank)).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    K = model.num_classes
    logits = torch.empty((B, K), dtype=torch.float32, device=dev)
    gathered = torch.empty((world * B, K), dtype=torch.float32, device=dev)

    def model_step():
        bound(x, out=logits)
        if world > 1:
            dist.all_gather_into_tensor(gathered, logits)

    for _ in range(args.warmup):
        model_step()
    ctx["barrier"]()
    total_ms = time_region(model_step, args.steps, dev, st)
    ctx["barrier"]()
    ms_step = total_ms / args.steps
    value = world * B * args.steps / (total_ms / 1e3)

    # per-kernel times from launch traces of the same forward
    agg, nl, per_launch = {}, 0, None
    reps = max(3, min(args.steps, 10))
    for _ in range(reps):
        _, launches = bound.forward_traced(x, out=logits)
        nl = len(launches)
        if per_launch is None:
            per_launch = [[kind, 0.0, nbytes] for kind, _, nbytes in launches]
        for i, (kind, ms, nbytes) in enumerate(launches):
            a = agg.setdefault(kind, [0, 0.0, 0.0])
            a[0] += 1; a[1] += ms; a[2] += nbytes
            per_launch[i][1] += ms / reps
    # every launch of one step in order: [kind, microseconds, algorithmic megabytes]
    launch_list = [[k, round(ms * 1e3, 1), round(nb / 1e6, 1)] for k, ms, nb in per_launch]
    peak, peak_src = peaks()
    kernels = {k: {"launches_per_step": a[0] // reps, "ms_per_step": a[1] / reps,
                   "algorithmic_bytes_per_step": a[2] / reps,
                   "achieved_GBps": (a[2] / reps) / (a[1] / reps / 1e3) / 1e9 if a[1] > 0 else None}
               for k, a in sorted(agg.items(), key=lambda kv: -kv[1][1])}
    top = next(iter(kernels))
    tk = kernels[top]
    kname = {"gemm": "gemm_bf16_kernel<false>", "conv_gemm": "gemm_bf16_kernel<true>",
             "dwconv7": "dwconv_tiled_kernel<7>", "dwconv3": "dwconv_tiled_kernel<3>",
             "layernorm": "layernorm_cl_kernel", "stem_conv": "stem_conv1_kernel",
             "spectral": "gated_spectral_cl_kernel", "mlp": "mlp_fused_kernel"}.get(top, top)
    roofline = {"bound": "hbm", "kernel": kname, "achieved": tk["achieved_GBps"], "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": tk["achieved_GBps"] / peak,
                "frac_of_nominal_8TBps": tk["achieved_GBps"] / 8000.0, "traffic": None,
                "algorithmic_bytes_per_launch": tk["algorithmic_bytes_per_step"] / tk["launches_per_step"],
                "ms_per_launch": tk["ms_per_step"] / tk["launches_per_step"],
                "launches_per_step": tk["launches_per_step"],
                "note": "all launches of the kernel in one step: sum of algorithmic bytes / sum of event times"}
    tr = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tr):
        with open(tr) as f:
            tj = json.load(f)
        per_img = tj.get(f"cfg5_{top}_dram_bytes_per_image")
        if per_img:
            roofline["traffic"] = per_img * B / tk["launches_per_step"]
    total_bytes = sum(k["algorithmic_bytes_per_step"] for k in kernels.values())
    model_hbm = {"algorithmic_bytes": total_bytes, "achieved": total_bytes / (ms_step / 1e3) / 1e9,
                 "unit": "GB/s", "frac": total_bytes / (ms_step / 1e3) / 1e9 / peak, "peak": peak,
                 "formula": "sum over the step's launches of inputs + outputs + weights"}

    e2e = None
    if not args.no_e2e:
        lh = torch.empty((B, K), dtype=torch.float32).pin_memory()
        # (a) one self-contained call per step: copies in chunks overlapped with compute inside the call
        for _ in range(max(1, min(args.warmup, 3))):
            bound.forward_host(x_host, lh)
        ctx["barrier"]()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            bound.forward_host(x_host, lh)             # returns after the logits arrived
        dt1 = shard.max_over_ranks(time.perf_counter() - t0, dev)
        # (b) the streaming loop: every call copies the NEXT step's images (a second pinned buffer)
        # while it computes its own, and returns after its logits arrived; one copy in and one
        # copy out per step inside the timed region
        x_host2 = x_host.clone().pin_memory()
        bufs = [x_host, x_host2]
        for i in range(max(2, min(args.warmup, 3))):
            bound.forward_host_pipelined(bufs[i & 1], bufs[(i + 1) & 1], lh)
        i0 = max(2, min(args.warmup, 3))
        ctx["barrier"]()
        t0 = time.perf_counter()
        for i in range(i0, i0 + args.steps):
            bound.forward_host_pipelined(bufs[i & 1], bufs[(i + 1) & 1], lh)
        dt = shard.max_over_ranks(time.perf_counter() - t0, dev)
        bound.close()
        e2e = {"value": world * B * args.steps / dt, "unit": "images/s",
               "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": lh.numel() * 4,
               "ms_per_step": 1e3 * dt / args.steps,
               "mode": "streaming loop: the host->device copy of step i+1 runs on a copy stream while "
                       "step i computes; every call returns after its own logits reached the host",
               "single_call_value": world * B * args.steps / dt1,
               "single_call_ms_per_step": 1e3 * dt1 / args.steps}

    sustained = None
    if ctx.get("sustain"):
        # the same loop for at least two seconds: the clock under sustained load, not a burst
        n_rep = max(1, int(2000.0 / max(ms_step * args.steps, 1e-3)) + 1)
        with ClockSampler(ctx["local"]) as cs:
            sus_ms = time_region(model_step, n_rep * args.steps, dev, st)
        sustained = {"value": world * B * n_rep * args.steps / (sus_ms / 1e3), "unit": "images/s",
                     "ms_per_step": sus_ms / (n_rep * args.steps), "seconds": sus_ms / 1e3,
                     "clocks": cs.summary()}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sb = min(cpu_sample_size(name), B)
        rate, dt, cores = cpu_model_rate(name, sb, reps=8)
        cpu = {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
               "sample": f"{sb} inputs of the {name} model, 8 repetitions ({dt:.2f} s each), torch-CPU "
                         f"(float32) restatement of the reference model"}
    m = wl["model"]
    return {
        "metric": metric_name(name), "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "model": "CSSM-SHViT s1 (embed_dims 64/128/256/384, depths 1/2/2/1)",
                   "block": "gated", "per_gpu_batch": B, "input": [wl["hw"], wl["hw"], 3],
                   "T": m["num_timesteps"], "kernel_sizes": list(m["kernel_sizes"]),
                   "gate_type": m["gate_type"], "num_classes": K,
                   "collective": "all-gather of the logits per step" if world > 1 else None,
                   "l2": "stage-0/1 activations (205 / 103 MB per tensor at batch 512) larger than the 126 MB L2"},
        "kernels": kernels, "launches": launch_list, "roofline": roofline, "model_hbm": model_hbm,
        "sustained": sustained, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": nl * args.steps,
    }


def run_simple(args, name, ctx):
    """One SimpleCSSM workload (cfg1..cfg4): device-timed model steps, last-frame-only variant,
    per-stage block times, roofline of the fused spectral kernel, end to end, CPU restatement."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from cssm_b200 import shard
    dev, st, world, rank = ctx["dev"], ctx["st"], ctx["world"], ctx["rank"]
    wl = WORKLOADS[name]
    barrier = ctx["barrier"]

    # model, weights, inputs (disjoint seeds per rank: every rank works on its own shard)
    B = wl["B"]
    if args.strong:
        if B % world:
            raise SystemExit(f"--strong: batch {B} does not divide over {world} ranks")
        B //= world
    model = make_model(name)
    x_np = make_inputs(name, B, seed0=1000 + B * rank)
    variables = model.init(0, x_np.shape)
    bound = model.bind(variables, dev)
    x_host = torch.from_numpy(np.ascontiguousarray(x_np)).pin_memory()
    x = x_host.to(dev)
    image_input = x.dim() == 4
    T = model.seq_len if image_input else x.shape[1]
    H, W = model.feature_hw(x.shape[-3], x.shape[-2])
    Cc = model.embed_dim
    gdn = model.cssm_type == "gdn"
    n_stem = 1 if model.stem_mode == "pathtracker" else model.stem_layers
    launches_per_step = n_stem + (9 if gdn else 5) + 2

    gathered = torch.empty((world * B, model.num_classes), dtype=torch.float32, device=dev)

    def model_step():
        """One forward of this rank's shard; with several ranks the logits are all-gathered
        (NCCL), the only collective of the run."""
        logits = bound(x)
        if world > 1:
            dist.all_gather_into_tensor(gathered, logits)
        return logits

    for _ in range(args.warmup):
        model_step()
    barrier()
    # ---- images on the device -> logits, all T block frames computed ----
    total_ms = time_region(model_step, args.steps, dev, st)
    barrier()
    ms_step = total_ms / args.steps
    value = world * B * args.steps / (total_ms / 1e3)
    # ---- the same with the block's last-frame-only entry point ----
    bound(x, last_frame_only=True)
    last_ms = time_region(lambda: bound(x, last_frame_only=True), args.steps, dev, st) / args.steps
    # ---- the block alone, stage by stage, on the stem features ----
    feat = bound.stem(x)
    feat5 = feat[:, None].expand(-1, T, -1, -1, -1).contiguous() if image_input else feat
    stem_ms = time_region(lambda: bound.stem(x, out=feat), args.steps, dev, st) / args.steps
    stage_ms, block_ms = block_stage_times(bound, feat5, args.steps, dev, st)
    del feat5

    # roofline of the fused spectral kernel
    peak, peak_src = peaks()
    per_unit = 20.0 * Cc * H * W if gdn else 12.0 * H * W * Cc      # bytes per (b,t)
    alg_bytes = per_unit * B * T
    achieved = alg_bytes / (stage_ms["spectral"] / 1e3) / 1e9
    kname = ("gdn_spectral_" if gdn else "gated_spectral_") + {64: "r64", 32: "r32"}.get(H, "generic")
    roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8TBps": achieved / 8000.0, "traffic": None,
                "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": stage_ms["spectral"]}
    tr = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tr):
        # DRAM bytes per unit from the committed ncu captures on the small workloads, scaled by
        # the units of this launch (traffic is proportional to them)
        with open(tr) as f:
            tj = json.load(f)
        if kname == "gated_spectral_r64" and tj.get("gated_spectral_r64_dram_bytes_per_plane_step"):
            roofline["traffic"] = tj["gated_spectral_r64_dram_bytes_per_plane_step"] * B * T * Cc
        elif gdn and tj.get(f"{kname}_dram_bytes_per_head_step"):
            roofline["traffic"] = tj[f"{kname}_dram_bytes_per_head_step"] * B * T * (Cc // model.delta_key_dim)

    # the whole block against the same peak: bytes a block with every stage fused to its
    # neighbours' GEMMs would still move (projection inputs / outputs and the fused kernel's planes)
    if gdn:
        blk_unit, blk_formula = 52.0, "(16 qkv_proj + 8 gate_proj + 20 spectral + 8 output_proj) * C*H*W per (b,t)"
    else:
        blk_unit, blk_formula = 32.0, "(12 in_proj + 12 spectral + 8 out_proj) * C*H*W per (b,t)"
    blk_bytes = blk_unit * Cc * H * W * B * T
    block_hbm = {"algorithmic_bytes": blk_bytes, "formula": blk_formula,
                 "achieved": blk_bytes / (block_ms / 1e3) / 1e9, "unit": "GB/s",
                 "frac": blk_bytes / (block_ms / 1e3) / 1e9 / peak, "peak": peak, "peak_source": peak_src}

    # ---- end to end: pinned host images -> host logits through the host-buffer entry point ----
    e2e = None
    if not args.no_e2e:
        lh = torch.empty((B, model.num_classes), dtype=torch.float32).pin_memory()

        def host_rate(last):
            for _ in range(max(1, min(args.warmup, 3))):
                bound.forward_host(x_host, lh, last_frame_only=last)
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                bound.forward_host(x_host, lh, last_frame_only=last)   # returns after the logits arrived
            return shard.max_over_ranks(time.perf_counter() - t0, dev)
        dt1 = host_rate(False)
        dt_last = host_rate(True)
        # the streaming loop: every call copies the NEXT step's batch (a second pinned buffer) while it
        # computes its own, and returns after its logits arrived
        x_host2 = x_host.clone().pin_memory()
        bufs = [x_host, x_host2]
        i0 = max(2, min(args.warmup, 3))
        for i in range(i0):
            bound.forward_host_pipelined(bufs[i & 1], bufs[(i + 1) & 1], lh)
        barrier()
        t0 = time.perf_counter()
        for i in range(i0, i0 + args.steps):
            bound.forward_host_pipelined(bufs[i & 1], bufs[(i + 1) & 1], lh)
        dt = shard.max_over_ranks(time.perf_counter() - t0, dev)
        bound.close()
        e2e = {"value": world * B * args.steps / dt, "unit": "images/s",
               "h2d_bytes_per_step": x_host.numel() * 4, "d2h_bytes_per_step": lh.numel() * 4,
               "ms_per_step": 1e3 * dt / args.steps,
               "mode": "streaming loop: the host->device copy of step i+1 runs on a copy stream while "
                       "step i computes; every call returns after its own logits reached the host",
               "single_call_value": world * B * args.steps / dt1,
               "last_frame_only_value": world * B * args.steps / dt_last}

    sustained = None
    if ctx.get("sustain"):
        n_rep = max(1, int(2000.0 / max(ms_step * args.steps, 1e-3)) + 1)
        with ClockSampler(ctx["local"]) as cs:
            sus_ms = time_region(model_step, n_rep * args.steps, dev, st)
        sustained = {"value": world * B * n_rep * args.steps / (sus_ms / 1e3), "unit": "images/s",
                     "ms_per_step": sus_ms / (n_rep * args.steps), "seconds": sus_ms / 1e3,
                     "clocks": cs.summary()}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sb = min(cpu_sample_size(name), B)
        reps = 4 if gdn else 8
        rate, dt, cores = cpu_model_rate(name, sb, reps=reps)
        cpu = {"value": rate, "unit": "images/s", "cores": cores, "kind": "port",
               "sample": f"{sb} inputs of the {name} model, {reps} repetitions ({dt:.2f} s "
                         f"each), torch-CPU restatement of the reference model"}

    return {
        "metric": metric_name(name), "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong" if args.strong else "weak",
        "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": name, "model": "SimpleCSSM depth 1", "block": model.cssm_type,
                   "per_gpu_batch": B, "input": list(x.shape[1:]), "T": T, "H": H, "W": W, "C": Cc,
                   "kernel_size": model.kernel_size, "gate_type": model.gate_type,
                   "pos_embed": model.pos_embed, "stem": model.stem_mode, "pool": model.pool_type,
                   "collective": "all-gather of the logits per step" if world > 1 else None,
                   "l2": "block activations (1.07 GB per tensor at cfg2-4) larger than the 126 MB L2"},
        "block": {"ms_per_step": block_ms, "stage_ms": stage_ms, "stem_ms": stem_ms, "hbm": block_hbm,
                  "value": world * B / (block_ms / 1e3), "unit": "images/s"},
        "stage_ms": stage_ms, "roofline": roofline,
        "last_frame_only": {"ms_per_step": last_ms, "value": world * B / (last_ms / 1e3),
                            "unit": "images/s"},
        "sustained": sustained, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps,
    }


HEADLINE = "cfg5"
ALSO = ["cfg1", "cfg2", "cfg3", "cfg4"]          # reported under "workloads" when no --workload is given


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help=f"one workload only (default: {HEADLINE} as the headline, then {', '.join(ALSO)})")
    ap.add_argument("--strong", action="store_true",
                    help="SimpleCSSM workloads: the workload's batch is the GLOBAL batch, split evenly "
                         "over the ranks (default: weak scaling, that batch per GPU)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sustain", action="store_true", help="skip the >= 2 s sustained loop (profiler runs)")
    args = ap.parse_args()
    single = args.workload is not None
    if not single:
        args.workload = HEADLINE
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: cssm_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # stdout carries the one JSON line: whatever NCCL logs (at the level the environment asked
        # for) goes to stderr unless the environment already names a file for it
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    st = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    ctx = dict(dev=dev, st=st, world=world, rank=rank, local=local, barrier=barrier, sustain=not args.no_sustain)
    run = lambda name: (run_shvit if is_shvit(name) else run_simple)(args, name, ctx)
    clk = ClockSampler(local)
    clk.__enter__()                       # sampled over the headline's timed regions
    line = run(args.workload)
    clk.__exit__(None, None, None)
    line["clocks"] = clk.summary()
    if not single and not args.strong:
        ctx["sustain"] = False
        line["workloads"] = {}
        for name in ALSO:
            r = run(name)
            line["workloads"][name] = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "dtype",
                                                        "config", "stage_ms", "block", "roofline",
                                                        "last_frame_only", "cpu_baseline", "e2e",
                                                        "gpu_launches") if k in r}
        if world > 1:
            # strong scaling of cfg2 beside the weak-scaling figures: its batch of 128 split over the ranks
            args.strong = True
            no_e2e, args.no_e2e = args.no_e2e, True
            r = run_simple(args, "cfg2", ctx)
            args.strong, args.no_e2e = False, no_e2e
            line["strong_scaling_cfg2"] = {"value": r["value"], "unit": "images/s", "ms_per_step": r["ms_per_step"],
                                           "global_batch": WORKLOADS["cfg2"]["B"], "n_gpus": world}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
