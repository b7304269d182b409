"""Performance sweep over the five benchmark configurations, one JSON line per case.

    python sweep.py [--quick] [--out results.jsonl]

The counterpart of the reference's perf sweeps (kernels/gemm/test/perf.py:62-77,
kernels/fmha/test/perf.py:100-113), which print a TFLOPS table per kernel index; here every
case is timed with CUDA events (about 30 ms of warm-up so the clocks have ramped, then the median of
5 repeats of >= 10 launches, alternating with the comparator; weights of memory-bound GEMMs are
rotated through 8 copies so they stream from HBM), next to the library comparators the
reference also uses as its kernels -1 / -2 (torch.matmul, scaled_dot_product_attention).
Rates: TFLOP/s = 2MNK/t (GEMM), 4*B*H*Sq*Skv*D/t, halved when causal (FMHA; the reference's
script does not halve); GB/s = algorithmic bytes / t.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "understanding-gpu-architecture-implications-on-llm-serving-workloads_b200")
if PKG not in sys.path:
    sys.path.insert(0, PKG)

from b200k import fmha, gemm, inputs  # noqa: E402


def _warm(fn, seconds=0.03):
    """Runs fn for about `seconds` of device time: after input generation the GPU sits at idle clocks,
    and a short kernel timed after a few calls only would be measured on the clock ramp."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    while total < seconds:
        e0.record()
        for _ in range(8):
            fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1) / 1e3


def _time_once(fn, n):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n / 1e3


def _time_pair(fn_a, fn_b, n, repeats=5):
    """Median seconds per call of two candidates, timed in alternation (a, b, a, b, ...) after both
    have warmed up, so that neither is favoured by the clocks the other left behind."""
    _warm(fn_a)
    _warm(fn_b)
    ta, tb = [], []
    for _ in range(repeats):
        ta.append(_time_once(fn_a, n))
        tb.append(_time_once(fn_b, n))
    return statistics.median(ta), statistics.median(tb)


def _time(fn, n, repeats=5):
    _warm(fn)
    return statistics.median(_time_once(fn, n) for _ in range(repeats))


def gemm_case(M, K, N, dtype, dev, n=20):
    copies = 8 if M <= 128 else 1
    a = inputs.device_randn16((M, K), 1, 1.0, dtype, dev)
    ws = [inputs.device_randn16((K, N), 2 + i, 0.02, dtype, dev) for i in range(copies)]
    out = torch.empty((M, N), dtype=dtype, device=dev)
    turn = [0]

    def ours():
        turn[0] = (turn[0] + 1) % copies
        gemm.gemm(a, ws[turn[0]], out=out)

    def lib():
        turn[0] = (turn[0] + 1) % copies
        torch.matmul(a, ws[turn[0]], out=out)

    n = n if M > 128 else 4 * n
    t, t_lib = _time_pair(ours, lib, n)
    flops, nbytes = 2.0 * M * N * K, 2.0 * (M * K + K * N + M * N)
    return {"path": "gemm", "M": M, "K": K, "N": N, "dtype": str(dtype).split(".")[-1], "us": t * 1e6,
            "tflops": flops / t / 1e12, "gbs": nbytes / t / 1e9, "cublas_tflops": flops / t_lib / 1e12,
            "cublas_gbs": nbytes / t_lib / 1e9}


def fmha_case(B, Hq, Hkv, S, D, causal, dtype, dev, n=10):
    q = inputs.device_randn16((B, Hq, S, D), 1, 1.0, dtype, dev)
    k = inputs.device_randn16((B, Hkv, S, D), 2, 1.0, dtype, dev)
    v = inputs.device_randn16((B, Hkv, S, D), 3, 1.0, dtype, dev)
    out = torch.empty_like(q)
    t, t_lib = _time_pair(lambda: fmha.fmha_fwd(q, k, v, causal=causal, out=out),
                          lambda: F.scaled_dot_product_attention(q, k, v, is_causal=causal, enable_gqa=True), n)
    flops = 4.0 * B * Hq * S * S * D * (0.5 if causal else 1.0)
    return {"path": "fmha", "B": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "causal": causal,
            "dtype": str(dtype).split(".")[-1], "us": t * 1e6, "tflops": flops / t / 1e12,
            "sdpa_tflops": flops / t_lib / 1e12}


def decode_case(dev, B=64, n=10):
    Hq, Hkv, Skv, D = 32, 8, 32768, 128
    lens = inputs.decode_lens(64)[:B].to(dev)
    q = inputs.device_randn16((B, Hq, 1, D), 7, 1.0, torch.float16, dev)
    k = inputs.device_randn16((B, Hkv, Skv, D), 8, 1.0, torch.float16, dev)
    v = inputs.device_randn16((B, Hkv, Skv, D), 9, 1.0, torch.float16, dev)
    out = torch.empty_like(q)
    ws = fmha.decode_workspace(B, Hq, Hkv, 1, Skv, D, 0, dev)
    t = _time(lambda: fmha.fmha_decode(q, k, v, kv_lens=lens, out=out, workspace=ws), n)
    nbytes = float(lens.sum().item()) * Hkv * D * 4 + 2.0 * B * Hq * D * 2
    return {"path": "decode", "B": B, "Hq": Hq, "Hkv": Hkv, "Skv": Skv, "D": D, "sum_len": int(lens.sum().item()),
            "us": t * 1e6, "gbs": nbytes / t / 1e9}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="one dtype, fewer shapes")
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default=None, choices=["gemm", "fmha", "decode"], help="one path only")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    sink = open(args.out, "w") if args.out else None

    def emit(rec):
        line = json.dumps(rec)
        print(line, flush=True)
        if sink:
            sink.write(line + "\n")
            sink.flush()

    want = lambda path: args.only in (None, path)
    if want("gemm"):
        emit(gemm_case(1024, 1024, 1024, torch.float16, dev, n=50))
        dtypes = [torch.bfloat16] if args.quick else [torch.bfloat16, torch.float16]
        for dtype in dtypes:
            for (K, N) in inputs.LLAMA7B_KN:
                for M in inputs.LLM_M + [64]:
                    emit(gemm_case(M, K, N, dtype, dev))
    if want("fmha"):
        emit(fmha_case(1, 32, 8, 4096, 128, True, torch.float16, dev, n=30))
        for D in (64, 128):
            for S in ((2048,) if args.quick else (1024, 2048, 8192)):
                for causal in (False, True):
                    emit(fmha_case(8, 32, 32, S, D, causal, torch.bfloat16, dev))
    if want("decode"):
        emit(decode_case(dev))
    if sink:
        sink.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
