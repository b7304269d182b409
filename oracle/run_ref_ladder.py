"""Times the reference's own kernel rungs (built for sm_100 by oracle/build_ref_ladder.py into
oracle/_ref/) on the current GPU, on the shapes of the reference's perf scripts
(kernels/gemm/test/perf.py:62-75: fp16 squares 2^10..2^13; kernels/fmha/test/perf.py:100-110:
B=1, 32/8 heads, d=128, causal, s = 2^10..2^14).  COMPARISON INFRASTRUCTURE ONLY.

    python oracle/run_ref_ladder.py            # prints one JSON line per (rung, size)

Runs in its own process: the reference libraries register the op namespaces gemm_unified /
fmha_unified, which the drop-in packages of this repo register too.  Only shapes the rungs
are written for are used (multiples of 128; the tensor-core rungs have no bounds checks), and
every result is compared with torch before it is timed.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _time(fn, n=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n / 1e3


def gemm_ladder():
    path = os.path.join(HERE, "_ref", "ref_gemm_unified.so")
    if not os.path.exists(path):
        return
    torch.ops.load_library(path)
    for rung in (8, 9, 10, 11):
        op = getattr(torch.ops.gemm_unified, f"finegemm_{rung}").default
        for e in (10, 11, 12, 13):
            n = 1 << e
            a = torch.randn(n, n, dtype=torch.half, device="cuda") * 0.1
            b = torch.randn(n, n, dtype=torch.half, device="cuda") * 0.1
            c = op(a, b)
            ref = a @ b
            err = float((c.float() - ref.float()).norm() / ref.float().norm())
            t = _time(lambda: op(a, b))
            print(json.dumps({"path": "gemm", "rung": rung, "n": n, "us": t * 1e6, "tflops": 2.0 * n ** 3 / t / 1e12,
                              "rel_err_vs_cublas": err}), flush=True)


def fmha_ladder():
    path = os.path.join(HERE, "_ref", "ref_fmha_unified.so")
    if not os.path.exists(path):
        return
    torch.ops.load_library(path)
    for rung in (2, 3, 4):
        op = getattr(torch.ops.fmha_unified, f"finefmha_{rung}").default
        for e in (10, 12, 14):
            s = 1 << e
            q = torch.randn(1, 32, s, 128, dtype=torch.half, device="cuda")
            k = torch.randn(1, 8, s, 128, dtype=torch.half, device="cuda")
            v = torch.randn(1, 8, s, 128, dtype=torch.half, device="cuda")
            o = op(q, k, v, True, False, s)
            ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            err = float((o.float() - ref.float()).abs().max())
            t = _time(lambda: op(q, k, v, True, False, s), n=5)
            print(json.dumps({"path": "fmha", "rung": rung, "s": s, "us": t * 1e6,
                              "tflops_executed": 2.0 * 32 * s * s * 128 / t / 1e12, "max_abs_vs_sdpa": err}), flush=True)


if __name__ == "__main__":
    which = sys.argv[1:] or ["gemm", "fmha"]
    if "gemm" in which:
        gemm_ladder()
    if "fmha" in which:
        fmha_ladder()
