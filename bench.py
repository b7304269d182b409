#!/usr/bin/env python
"""Benchmark of the B200 kernels: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline metric: TFLOP/s of the LLM-projection GEMM (bf16, M=8192 tokens against
the Llama-2-7B-shaped 4096x11008 weight, fp32 accumulate), the largest single-GPU
case of the GEMM sweep.  A step is one pass of that GEMM over synthetic
operands (A ~ N(0,1), W ~ N(0,0.02)).  `value` is timed with the operands resident
in HBM; `e2e` times the reference-facing call `gemm_unified.ops.fine_gemm` with
HOST operands (pinned), host->device and device->host copies inside the timed
region.  Operands + output are 334 MB per step, larger than the 126 MB L2.

The same line carries, under "extra", the causal FMHA prefill configuration
(fp16, B=1, 32/8 heads, s=4096, d=128; TFLOP/s with the causal half counted
once) and the split-KV decode configuration (fp16, B=64, s_q=1, 32/8 heads,
d=128, KV lengths uniform in [512, 32768]; GB/s of valid K+V bytes).

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank owns
one N-tile slab of a weight that is N times wider (per-GPU work fixed, "weak"),
no data-path collective; the time is the max over ranks.

--impl reference times the reference's CPU path for the same math (fp32
torch.matmul on the host cores: the function the reference's own check uses,
kernels/gemm/test/correct.py:9-16) on a bounded row slab of the same GEMM.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "understanding-gpu-architecture-implications-on-llm-serving-workloads_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

M, K, N = 8192, 4096, 11008
WORKLOAD = f"llm_projection_gemm_bf16_M{M}_K{K}_N{N}"
METRIC = "gemm_tflops"
UNIT = "TFLOP/s"
FLOPS_PER_STEP = 2.0 * M * N * K
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM kernel on this
# workload, from the ncu capture summarised in profiles/ (None until captured)
NCU_TRAFFIC_BYTES = 697283072  # 526.9 MB read + 170.4 MB written (ncu capture summarised under profiles/)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU every few
    milliseconds through NVML while the timed region runs (the same counters
    `nvidia-smi --query-gpu=clocks.sm,clocks_event_reasons.*` prints; a polling
    thread is used because the timed region is shorter than nvidia-smi's period)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.mask = [], 0
        self.sm_max = None
        self._stop = threading.Event()
        self.thread = None
        self.marks = {}

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                ids = [x for x in visible.split(",") if x.strip()]
                if self.index < len(ids) and ids[self.index].strip().isdigit():
                    idx = int(ids[self.index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def mark(self, name: str):
        self.marks[name] = time.perf_counter()

    def _poll(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    reasons = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    reasons = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        if not self.thread:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": "unavailable"}
        self._stop.set()
        self.thread.join(timeout=2)
        t0, t1 = self.marks.get("begin", 0.0), self.marks.get("end", float("inf"))
        inside = [(m, r) for (t, m, r) in self.samples if t0 <= t <= t1]
        mask = 0
        for _, r in inside:
            mask |= r
        reasons = sorted(name for name, bit in self.REASONS.items() if mask & bit)
        return {"sm_mhz": statistics.median(m for m, _ in inside) if inside else None, "sm_max_mhz": self.sm_max,
                "reasons": reasons, "samples": len(inside), "source": "nvml polling during the timed region"}


def warm_for(fn, seconds: float) -> None:
    """Calls fn until about `seconds` of device time have passed: after host-side set-up (input
    generation, copies) the GPU has dropped to idle clocks, and a sub-millisecond kernel timed right
    after a handful of warm-up calls is measured on the ramp, not at the clocks it runs at in a job."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    while total < seconds:
        e0.record()
        for _ in range(8):
            fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1) / 1e3


def time_cuda(fn, steps: int, warmup: int, barrier=None, sampler=None, warm_seconds: float = 0.0) -> float:
    """Seconds for `steps` calls of fn, CUDA events on the current stream, after warm-up."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if warm_seconds > 0:
        warm_for(fn, warm_seconds)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark("begin")
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark("end")
    if barrier:
        barrier()
    return e0.elapsed_time(e1) / 1e3


# ------------------------------------------------------------------ CPU baseline / reference arm
def cpu_gemm_sample(target_seconds: float, repeats: int = 1):
    """Times the oracle's fp32 CPU matmul on a row slab of the same GEMM (full K and N)
    sized for about `target_seconds`; returns (TFLOP/s, threads, description)."""
    from oracle import oracle
    from b200k import inputs
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16)
    probe_rows = 64
    a = torch.randn(probe_rows, K, generator=g).to(torch.bfloat16)
    oracle.gemm_ref(a, w)  # warm-up (thread pool, page faults)
    t0 = time.perf_counter()
    oracle.gemm_ref(a, w)
    probe = max(time.perf_counter() - t0, 1e-4)
    rows = int(min(M, max(probe_rows, probe_rows * target_seconds / probe)))
    rows = max(64, rows // 64 * 64)
    a = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.gemm_ref(a, w)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    tflops = 2.0 * rows * N * K / best / 1e12
    del inputs
    return tflops, threads, f"fp32 torch.matmul on CPU, {rows} of {M} rows x full K={K}, N={N} (bf16-rounded operands widened to fp32)", rows, best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps, warmup = args.steps, args.warmup
    from oracle import oracle
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16)
    # slab sized so that one step is ~1.5 s of CPU work
    tflops0, threads, _, _, _ = cpu_gemm_sample(1.5)
    rows = int(min(M, max(64, (1.5 * tflops0 * 1e12 / (2.0 * N * K)) // 64 * 64)))
    a = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    for _ in range(warmup):
        oracle.gemm_ref(a, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.gemm_ref(a, w)
    dt = time.perf_counter() - t0
    value = 2.0 * rows * N * K * steps / dt / 1e12
    sample = f"each step: fp32 torch.matmul on CPU of {rows} of {M} rows x full K={K}, N={N}"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_rows": rows},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------ small cases for ncu captures
def run_profile_case(args):
    """Runs ONE hot path a few times (inputs larger than L2, at most ~2 GB on the device, nothing
    else on the GPU) so that a profiler capture of it ends by itself; prints a short JSON line."""
    from b200k import _lib, fmha, gemm, inputs
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    case, n = args.profile_case, max(1, args.steps)
    if case == "gemm":
        a = inputs.device_randn16((M, K), 100, 1.0, torch.bfloat16, dev)
        w = inputs.device_randn16((K, N), 200, 0.02, torch.bfloat16, dev)
        c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        fn = lambda: gemm.gemm(a, w, out=c, variant=args.variant)
        work, unit = FLOPS_PER_STEP / 1e12, "TFLOP/s"
    elif case == "fmha":
        q, k, v = inputs.fmha_c3(dev)
        o = torch.empty_like(q)
        fn = lambda: fmha.fmha_fwd(q, k, v, causal=True, out=o)
        work, unit = 4.0 * 32 * 4096 * 4096 * 128 * 0.5 / 1e12, "TFLOP/s"
    elif case == "decode":
        B, Hq, Hkv, Skv, D = 16, 32, 8, 32768, 128   # a quarter of the batch: 2 GiB of K+V
        lens = inputs.decode_lens(64)[:B].to(dev)
        q = inputs.device_randn16((B, Hq, 1, D), 7, 1.0, torch.float16, dev)
        k = inputs.device_randn16((B, Hkv, Skv, D), 8, 1.0, torch.float16, dev)
        v = inputs.device_randn16((B, Hkv, Skv, D), 9, 1.0, torch.float16, dev)
        o = torch.empty_like(q)
        ws = fmha.decode_workspace(B, Hq, Hkv, 1, Skv, D, 0, dev)
        fn = lambda: fmha.fmha_decode(q, k, v, kv_lens=lens, out=o, workspace=ws)
        work, unit = (float(lens.sum().item()) * Hkv * D * 4 + 2.0 * B * Hq * D * 2) / 1e9, "GB/s"
    elif case == "decode_short":
        # a large batch of short sequences: every sequence unsplit, the split kernel walks strided lists of
        # (sequence, head) pairs and writes O itself; 0.5 GiB of K+V
        B, Hq, Hkv, Skv, D = 512, 32, 8, 256, 128
        lens = torch.full((B,), Skv, dtype=torch.int32, device=dev)
        q = inputs.device_randn16((B, Hq, 1, D), 7, 1.0, torch.bfloat16, dev)
        k = inputs.device_randn16((B, Hkv, Skv, D), 8, 1.0, torch.bfloat16, dev)
        v = inputs.device_randn16((B, Hkv, Skv, D), 9, 1.0, torch.bfloat16, dev)
        o = torch.empty_like(q)
        ws = fmha.decode_workspace(B, Hq, Hkv, 1, Skv, D, 0, dev)
        fn = lambda: fmha.fmha_decode(q, k, v, kv_lens=lens, out=o, workspace=ws)
        work, unit = (float(B) * Skv * Hkv * D * 4 + 2.0 * B * Hq * D * 2) / 1e9, "GB/s"
    elif case == "skinny":
        # the decode pairing: 64 rows against the 4096 x 11008 weight, four copies in rotation so that
        # every launch streams its weight from HBM (one copy, 90 MB, would sit in the 126 MB L2)
        Ms, Ks, Ns = 64, 4096, 11008
        xs = inputs.device_randn16((Ms, Ks), 11, 1.0, torch.bfloat16, dev)
        wts = [inputs.device_randn16((Ks, Ns), 20 + t, 0.02, torch.bfloat16, dev) for t in range(4)]
        cs = torch.empty((Ms, Ns), dtype=torch.bfloat16, device=dev)
        turn = [0]

        def fn():
            turn[0] = (turn[0] + 1) % len(wts)
            gemm.gemm(xs, wts[turn[0]], out=cs)
        work, unit = 2.0 * (Ks * Ns + Ms * Ks + Ms * Ns) / 1e9, "GB/s"
    else:
        raise SystemExit(f"unknown --profile-case {case}")
    secs = time_cuda(fn, n, max(1, args.warmup))
    code, detail = _lib.device_status()
    print(json.dumps({"profile_case": case, "launch_ms": secs / n * 1e3, "rate": work * n / secs, "unit": unit,
                      "device_status": code}), flush=True)
    return 0 if code == 0 else 1


# ------------------------------------------------------------------ our arm
def run_ours(args):
    import torch.distributed as dist
    from b200k import _lib, fmha, gemm, inputs
    import gemm_unified

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()  # fail loudly here if the extension is missing

    def barrier():
        if distributed:
            dist.barrier()

    def max_over_ranks(seconds: float) -> float:
        if not distributed:
            return seconds
        t = torch.tensor([seconds], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    steps, warmup = args.steps, max(args.warmup, 3)
    peaks = measured_peaks()

    # ---- headline GEMM: rank r owns column slab r of a weight N*world wide (weak scaling) ----
    a = inputs.device_randn16((M, K), 100 + rank, 1.0, torch.bfloat16, dev)
    w = inputs.device_randn16((K, N), 200 + rank, 0.02, torch.bfloat16, dev)
    c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

    def step():
        gemm.gemm(a, w, out=c)

    sampler = ClockSampler(local_rank)
    launches0 = _lib.launch_count()
    if rank == 0:
        sampler.start()
    secs = max_over_ranks(time_cuda(step, steps, warmup, barrier, sampler if rank == 0 else None))
    launches = _lib.launch_count() - launches0 - warmup
    clocks = sampler.stop() if rank == 0 else None
    code, detail = _lib.device_status()
    if code != 0:
        raise SystemExit(f"device status {code} detail {detail:#x} after the timed region")
    value = world * FLOPS_PER_STEP * steps / secs / 1e12
    kernel_tflops = FLOPS_PER_STEP * steps / secs / 1e12  # per GPU == the kernel's own rate

    # ---- e2e: reference-facing op, host operands, copies inside the timed region ----
    a_h = a.cpu().pin_memory()
    w_h = w.cpu().pin_memory()
    c_h = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    # Pipelined over three buffer sets: step s copies its operands in on one stream while step s-1 computes on a
    # second and step s-2's result is read back on a third, so the PCIe directions and the GPU
    # overlap; every step still moves all of its inputs and its whole result.
    nbuf = 3
    a_d = [torch.empty_like(a) for _ in range(nbuf)]
    w_d = [torch.empty_like(w) for _ in range(nbuf)]
    c_hs = [c_h] + [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(nbuf - 1)]
    st_in, st_run, st_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_run(nsteps):
        main = torch.cuda.current_stream()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(main)
        for st in (st_in, st_run, st_out):
            st.wait_event(start)
        ran = [None] * nbuf      # compute finished with buffer set i
        read = [None] * nbuf     # result of buffer set i is back on the host
        keep = [None] * nbuf
        for step_i in range(nsteps):
            i = step_i % nbuf
            with torch.cuda.stream(st_in):
                if ran[i] is not None:
                    st_in.wait_event(ran[i])          # operands of set i no longer in use
                a_d[i].copy_(a_h, non_blocking=True)
                w_d[i].copy_(w_h, non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(st_in)
            with torch.cuda.stream(st_run):
                st_run.wait_event(loaded)
                out = gemm_unified.ops.fine_gemm(a_d[i], w_d[i], 12)
                ran[i] = torch.cuda.Event()
                ran[i].record(st_run)
            with torch.cuda.stream(st_out):
                st_out.wait_event(ran[i])
                if read[i] is not None:
                    st_out.wait_event(read[i])
                out.record_stream(st_out)
                c_hs[i].copy_(out, non_blocking=True)
                read[i] = torch.cuda.Event()
                read[i].record(st_out)
            keep[i] = out
        for st in (st_in, st_run, st_out):
            done = torch.cuda.Event()
            done.record(st)
            main.wait_event(done)
        stop.record(main)
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / 1e3

    e2e_steps = max(4, min(steps, 12))
    e2e_run(4)  # warm-up
    barrier()
    e2e_secs = max_over_ranks(e2e_run(e2e_steps))
    barrier()
    e2e_value = world * FLOPS_PER_STEP * e2e_steps / e2e_secs / 1e12
    h2d = a_h.numel() * 2 + w_h.numel() * 2
    d2h = c_h.numel() * 2
    del a_h, w_h, c_h, c_hs, a_d, w_d

    # ---- extra: FMHA prefill (causal, s=4096) and split-KV decode ----
    extra = {}
    try:
        q, k, v = inputs.fmha_c3(dev)
        o = torch.empty_like(q)
        fsteps = max(steps, 50)
        fsecs = max_over_ranks(time_cuda(lambda: fmha.fmha_fwd(q, k, v, causal=True, out=o), fsteps, warmup, barrier,
                                         warm_seconds=0.03))
        fflops = 4.0 * 1 * 32 * 4096 * 4096 * 128 * 0.5
        tf = world * fflops * fsteps / fsecs / 1e12
        extra["fmha_prefill"] = {
            "workload": "causal_fmha_fp16_B1_H32_8_S4096_D128", "value": tf, "unit": "TFLOP/s",
            "ms": fsecs / fsteps * 1e3, "flops_convention": "executed (causal half counted once)",
            "reference_convention_tflops": 2 * tf,
            "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": tf / world / peaks["tflops"], "traffic": None}}
        del q, k, v, o
        B, Hq, Hkv, Skv, D = 64, 32, 8, 32768, 128
        lens = inputs.decode_lens(B).to(dev)
        qd = inputs.device_randn16((B, Hq, 1, D), 7, 1.0, torch.float16, dev)
        kd = inputs.device_randn16((B, Hkv, Skv, D), 8, 1.0, torch.float16, dev)
        vd = inputs.device_randn16((B, Hkv, Skv, D), 9, 1.0, torch.float16, dev)
        od = torch.empty_like(qd)
        ws = fmha.decode_workspace(B, Hq, Hkv, 1, Skv, D, 0, dev)
        dsteps = max(steps, 10)
        dsecs = max_over_ranks(time_cuda(
            lambda: fmha.fmha_decode(qd, kd, vd, kv_lens=lens, out=od, workspace=ws), dsteps, warmup, barrier,
            warm_seconds=0.03))
        dbytes = float(lens.sum().item()) * Hkv * D * 2 * 2 + 2.0 * B * Hq * D * 2
        gbs = world * dbytes * dsteps / dsecs / 1e9
        extra["decode_splitkv"] = {
            "workload": "decode_fp16_B64_Sq1_H32_8_D128_kvlen_U512_32768", "value": gbs, "unit": "GB/s",
            "ms": dsecs / dsteps * 1e3, "bytes": "valid K+V once, q and o once",
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / world / peaks["hbm_gbs"], "traffic": None}}
        del qd, kd, vd, od, ws
        # skinny GEMM paired with the decode configuration: M=64 tokens against the 4096x11008 weight,
        # 8 weight copies rotated so that the weight is streamed from HBM, not from L2
        Ms, Ks, Ns = 64, 4096, 11008
        xs = inputs.device_randn16((Ms, Ks), 11, 1.0, torch.bfloat16, dev)
        wts = [inputs.device_randn16((Ks, Ns), 20 + t, 0.02, torch.bfloat16, dev) for t in range(8)]
        cs = torch.empty((Ms, Ns), dtype=torch.bfloat16, device=dev)
        turn = [0]

        def skinny_step():
            turn[0] = (turn[0] + 1) % len(wts)
            gemm.gemm(xs, wts[turn[0]], out=cs)

        ssteps = max(steps, 200)
        ssecs = max_over_ranks(time_cuda(skinny_step, ssteps, warmup, barrier, warm_seconds=0.03))
        sbytes = 2.0 * (Ks * Ns + Ms * Ks + Ms * Ns)
        sgbs = world * sbytes * ssteps / ssecs / 1e9
        # the same launches replayed from a CUDA graph (as a serving loop would issue them): device time
        # without the per-call host overhead of the Python binding
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(len(wts)):
                skinny_step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(len(wts)):
                skinny_step()
        gsteps = max(4, ssteps // len(wts))
        gsecs = max_over_ranks(time_cuda(graph.replay, gsteps, 3, barrier)) / len(wts)
        ggbs = world * sbytes * gsteps / gsecs / 1e9
        extra["skinny_gemm"] = {
            "workload": "gemm_bf16_M64_K4096_N11008", "value": ggbs, "unit": "GB/s", "ms": gsecs / gsteps * 1e3,
            "note": "launches replayed from a CUDA graph, weights rotated through 8 copies (HBM-resident, not L2)",
            "per_call_from_python": {"value": sgbs, "unit": "GB/s", "ms": ssecs / ssteps * 1e3,
                                     "note": "one launch per call through the ctypes binding, host overhead inside"},
            "roofline": {"bound": "hbm", "achieved": ggbs / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ggbs / world / peaks["hbm_gbs"], "traffic": 94146304}}
        del graph
        del xs, wts, cs
    except Exception as exc:  # the headline number stands even if an extra fails
        extra["error"] = repr(exc)[:300]

    # ---- strong scaling of the attention paths: a FIXED problem sharded over the ranks ----
    # prefill: bf16, B=8, 32 heads (MHA), s=2048, d=128, causal, (batch, head) pairs dealt to the ranks;
    # decode: the 64-sequence batch above, sequences balanced by total KV length.  No collective: the
    # output stays sharded; the time is the slowest rank's.
    try:
        from b200k import shard as _shard
        Bp, Hp, Sp, Dp = 8, 32, 2048, 128
        mine = _shard.head_shards(Bp, Hp, Hp, world)[rank]
        parts = []
        for (bb, h0, nh) in mine:
            qs = inputs.device_randn16((1, nh, Sp, Dp), 300 + bb * Hp + h0, 1.0, torch.bfloat16, dev)
            parts.append((qs, torch.randn_like(qs), torch.randn_like(qs), torch.empty_like(qs)))

        def prefill_shard():
            for (q_, k_, v_, o_) in parts:
                fmha.fmha_fwd(q_, k_, v_, causal=True, out=o_)

        psteps = max(steps, 10)
        psecs = max_over_ranks(time_cuda(prefill_shard, psteps, warmup, barrier))
        pflops = 4.0 * Bp * Hp * Sp * Sp * Dp * 0.5
        extra["fmha_prefill_sharded"] = {
            "workload": "causal_fmha_bf16_B8_H32_S2048_D128 over all ranks ((batch, head) shards)",
            "value": pflops * psteps / psecs / 1e12, "unit": "TFLOP/s", "ms": psecs / psteps * 1e3,
            "scaling": "strong", "launches_per_rank": len(parts)}
        del parts
        Bd, Hqd, Hkvd, Skvd, Dd = 64, 32, 8, 32768, 128
        all_lens = inputs.decode_lens(Bd)
        idx = _shard.balance_sequences(all_lens.tolist(), world)[rank]
        nb_ = len(idx)
        lens_r = all_lens[idx].to(dev)
        qd = inputs.device_randn16((nb_, Hqd, 1, Dd), 7, 1.0, torch.float16, dev)
        kd = inputs.device_randn16((nb_, Hkvd, Skvd, Dd), 8, 1.0, torch.float16, dev)
        vd = inputs.device_randn16((nb_, Hkvd, Skvd, Dd), 9, 1.0, torch.float16, dev)
        od = torch.empty_like(qd)
        wsd = fmha.decode_workspace(nb_, Hqd, Hkvd, 1, Skvd, Dd, 0, dev)
        dsteps2 = max(steps, 10)
        dsecs2 = max_over_ranks(time_cuda(
            lambda: fmha.fmha_decode(qd, kd, vd, kv_lens=lens_r, out=od, workspace=wsd), dsteps2, warmup, barrier))
        dbytes2 = float(all_lens.sum().item()) * Hkvd * Dd * 4 + 2.0 * Bd * Hqd * Dd * 2
        extra["decode_sharded"] = {
            "workload": "the 64-sequence decode batch over all ranks (sequences balanced by KV length)",
            "value": dbytes2 * dsteps2 / dsecs2 / 1e9, "unit": "GB/s", "ms": dsecs2 / dsteps2 * 1e3,
            "scaling": "strong", "sequences_this_rank": nb_}
        del qd, kd, vd, od, wsd
    except Exception as exc:
        extra["sharded_error"] = repr(exc)[:300]

    # ---- N > 1: the one collective of the GEMM path, reassembling a column-sharded product ----
    if distributed:
        try:
            from b200k import shard
            slabs = shard.gemm_column_slabs(N, world)
            s0, e0 = slabs[rank]
            w_slab = w[:, s0:e0]

            def nccl_step():
                shard.all_gather_columns(gemm.gemm(a, w_slab), slabs)

            gsteps = max(5, min(steps, 20))
            nccl_secs = max_over_ranks(time_cuda(nccl_step, gsteps, 3, barrier))
            fused = shard.FusedAllGatherGemm(M, N, torch.bfloat16, dev)
            fused_secs = max_over_ranks(time_cuda(lambda: fused(a, w_slab), gsteps, 3, barrier))
            extra["gemm_allgather_strong"] = {
                "workload": f"C[{M},{N}] = A . W with W column-sharded over {world} GPUs, full C on every rank",
                "nccl_ms": nccl_secs / gsteps * 1e3, "fused_epilogue_ms": fused_secs / gsteps * 1e3,
                "tflops_fused": FLOPS_PER_STEP * gsteps / fused_secs / 1e12,
                "note": "nccl = local slab GEMM + all_gather_into_tensor + column reassembly; fused = epilogue TMA "
                        "stores into all ranks' symmetric buffers + symmetric-memory barrier"}
        except Exception as exc:
            extra["gemm_allgather_strong"] = {"error": repr(exc)[:300]}

    # ---- CPU baseline on rank 0 at N=1 ----
    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        tflops, threads, sample, _, _ = cpu_gemm_sample(10.0)
        cpu = {"value": tflops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        algorithmic = "flops"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": secs / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "accumulate": "f32", "l2": "operands+output 334 MB per step > 126 MB L2",
                       "sharding": "rank r owns N-tile slab r of a weight N*n_gpus wide; no data-path collective",
                       "peak_source": peaks["source"]},
            "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": kernel_tflops / peaks["tflops"], "traffic": NCU_TRAFFIC_BYTES,
                         "algorithmic": algorithmic, "frac_of_nominal_2250": kernel_tflops / 2250.0},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "gemm_unified.ops.fine_gemm(a, b, 12)", "pipelining": "3 buffer sets, copy-in / compute / copy-out streams"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-case", default=None, choices=["gemm", "fmha", "decode", "decode_short", "skinny"],
                    help="run only this path on a capture-sized case (for ncu); prints its own short line")
    ap.add_argument("--variant", type=int, default=0, help="GEMM kernel variant for --profile-case gemm")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "ours" and args.gpus != world and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with --nproc-per-node {args.gpus} "
                         f"(WORLD_SIZE is {world})")
    if args.profile_case:
        return run_profile_case(args)
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
