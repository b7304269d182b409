"""bench.py's reference arm runs without a GPU (it times the CPU path on the host cores) and prints
the contract's JSON line; the library arm refuses to run without a GPU instead of falling back."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=300, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=ROOT, env=env)


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


def test_reference_arm_under_a_multi_rank_launcher_uses_all_cores_and_the_same_sample():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: rank 0 must still time the CPU
    path on every core it may use and on the same rows as at N=1 (same config object), and the other
    ranks must exit 0 without printing."""
    base = dict(os.environ, OMP_NUM_THREADS="1", WORLD_SIZE="4", LOCAL_RANK="0")
    p0 = _run("--impl", "reference", "--gpus", "4", "--steps", "1", "--warmup", "0", env=dict(base, RANK="0"))
    p1 = _run("--impl", "reference", "--gpus", "4", "--steps", "1", "--warmup", "0", env=dict(base, RANK="1"))
    assert p0.returncode == 0 and p1.returncode == 0 and p1.stdout.strip() == ""
    line = json.loads([l for l in p0.stdout.splitlines() if l.startswith("{")][-1])
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    single = json.loads([l for l in _run("--impl", "reference", "--steps", "1", "--warmup", "0").stdout.splitlines()
                         if l.startswith("{")][-1])
    assert line["cpu_baseline"]["sample_rows"] == single["cpu_baseline"]["sample_rows"]
    assert line["n_gpus"] == 4 and line["config"]["workload"] == single["config"]["workload"]


def test_library_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return  # on a GPU box the arm runs; the GPU suite covers it
    p = _run("--steps", "1", "--warmup", "1", "--no-cpu-baseline", timeout=120)
    assert p.returncode != 0
    assert "{\"metric\"" not in p.stdout
