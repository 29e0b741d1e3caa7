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
    assert d["config"]["workload"] == "cfg2"


def test_workloads_match_baseline_configs():
    sys.path.insert(0, ROOT)
    import bench
    w = bench.WORKLOADS
    assert w["cfg2"]["B"] == 128 and w["cfg2"]["T"] == 8 and w["cfg2"]["kernel_size"] == 11
    assert w["cfg2"]["gate_type"] == "factored" and w["cfg2"]["C"] == 64
    assert w["cfg3"]["block"] == "gdn" and w["cfg3"]["delta_key_dim"] == 4 and w["cfg3"]["qkv_conv_size"] == 5
    assert w["cfg4"]["T"] == 32 and w["cfg4"]["H"] == 32
