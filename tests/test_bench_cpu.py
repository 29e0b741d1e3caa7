"""CPU test of the reference arm of bench.py: it must run without a GPU and print one JSON line
with the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_json():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = out.stdout.strip().splitlines()[-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and d["unit"] == "images/s" and d["value"] > 0
    for k in ("metric", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert k in d, k
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
    assert d["config"]["workload"] == "cfg5" and d["dtype"] == "bf16"     # the default headline


def test_workloads_match_baseline_configs():
    sys.path.insert(0, ROOT)
    import bench
    w = bench.WORKLOADS
    m2 = w["cfg2"]["model"]
    assert w["cfg2"]["B"] == 128 and m2["seq_len"] == 8 and m2["kernel_size"] == 11
    assert m2["gate_type"] == "factored" and m2["embed_dim"] == 64 and m2["stem_layers"] == 1
    assert m2["cssm_type"] == "gated" and m2["pool_type"] == "max" and m2["num_classes"] == 2
    m3 = w["cfg3"]["model"]
    assert m3["cssm_type"] == "gdn" and m3["delta_key_dim"] == 4 and m3["qkv_conv_size"] == 5
    assert m3["pos_embed"] == "mrope" and m3["output_norm"] == "rms"
    m4 = w["cfg4"]["model"]
    assert m4["cssm_type"] == "gdn" and m4["stem_mode"] == "pathtracker" and w["cfg4"]["data"] == "dots"
    m5 = w["cfg5"]["model"]
    assert w["cfg5"]["B"] == 512 and m5["num_timesteps"] == 1 and m5["num_classes"] == 1000
    assert tuple(m5["embed_dims"]) == (64, 128, 256, 384) and tuple(m5["depths"]) == (1, 2, 2, 1)
    assert tuple(m5["kernel_sizes"]) == (1, 1, 1, 1) and m5["short_conv_spatial_size"] == 0
    assert bench.make_inputs("cfg5", 2, seed0=1).shape == (2, 224, 224, 3)
    x = bench.make_inputs("cfg4", 2, seed0=1)
    assert x.shape == (2, 32, 32, 32, 3)
    assert bench.make_inputs("cfg2", 1, seed0=1).shape == (1, 128, 128, 1)


def test_simple_reference_arms_run():
    for wl in ("cfg2", "cfg4"):
        out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                              "--workload", wl, "--steps", "1", "--warmup", "0"],
                             capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert out.returncode == 0, out.stderr[-2000:]
        d = json.loads(out.stdout.strip().splitlines()[-1])
        assert d["impl"] == "reference" and d["value"] > 0 and d["config"]["workload"] == wl
