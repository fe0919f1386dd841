"""CPU: the reference arm of bench.py runs without a GPU and prints one JSON line with the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         check=True, capture_output=True, text=True, cwd=ROOT, timeout=300).stdout.strip().splitlines()
    line = json.loads(out[-1])
    assert line["impl"] == "reference" and line["metric"] == "seglinear_gemm_tops" and line["unit"] == "TOPS"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype", "data",
                "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["value"] > 0 and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["kind"] in ("port", "reference")
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"]


def test_workloads_and_flags_parse():
    help_text = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], check=True, capture_output=True, text=True,
                               cwd=ROOT, timeout=120).stdout
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--workload", "--fused-gather", "--sweep-nk", "--kernel-rows"):
        assert flag in help_text, flag
