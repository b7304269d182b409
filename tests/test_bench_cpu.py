"""bench.py's reference arm runs without a GPU (it times the CPU path on the host cores) and prints
the contract's JSON line; the library arm refuses to run without a GPU instead of falling back."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=300):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=ROOT)


def test_reference_arm_prints_the_contract_line():
    p = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["unit"] == "TFLOP/s" and line["value"] > 0 and line["steps"] == 1 and line["warmup"] == 0
    assert line["config"]["workload"].startswith("llm_projection_gemm_bf16_M8192_K4096_N11008")
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "rows" in cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}


def test_library_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return  # on a GPU box the arm runs; the GPU suite covers it
    p = _run("--steps", "1", "--warmup", "1", "--no-cpu-baseline", timeout=120)
    assert p.returncode != 0
    assert "{\"metric\"" not in p.stdout
