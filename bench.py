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

With N > 1 (launched by torch.distributed.run, one rank per GPU) the SAME GEMM is
sharded: rank r owns N-tile column slab r of the one 4096x11008 weight, the
activations are replicated, the product stays column-sharded (no data-path
collective); total work is fixed ("strong" scaling), the time is the slowest
rank's.  The all-gather that reassembles the full product on every rank (NCCL,
and fused into the GEMM epilogue) is timed separately under "extra", as are the
per-GPU replica rate ("gemm_weak"), the FMHA prefill and split-KV decode
configurations with their own rooflines, CPU baselines and end-to-end numbers,
a sustained (power-capped) run of the headline GEMM, and bit-exactness of the
sharded results against unsharded ones computed in the same run.

--impl reference times the reference's CPU path for the same math (fp32
torch.matmul on the host cores: the function the reference's own check uses,
kernels/gemm/test/correct.py:9-16) on a fixed row slab of the same GEMM, with
all the host threads the process may use.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
# rows of the GEMM one step of the CPU arm computes (full K and N): a fixed, bounded sample
REFERENCE_SAMPLE_ROWS = 2048
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM kernel on this
# workload, from the ncu capture summarised in profiles/
NCU_TRAFFIC_BYTES = 534907904  # 369.1 MB read + 165.8 MB written


def bench_config(n_gpus: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "M": M, "K": K, "N": N, "accumulate": "f32",
            "l2": "operands+output 334 MB per step > 126 MB L2",
            "sharding": "none" if n_gpus == 1 else
            f"rank r owns N-tile column slab r of the weight ({n_gpus} slabs), activations replicated, "
            "product left column-sharded; no data-path collective"}


def host_threads() -> int:
    """Host cores this process may run on (its affinity mask, not the machine's core count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", 0)) or None,
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU every few
    milliseconds through NVML while the timed region runs (the same counters
    `nvidia-smi --query-gpu=clocks.sm,clocks_event_reasons.*` prints; a polling
    thread is used because the timed region is shorter than nvidia-smi's period)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples = []
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

    def window(self, t0: float, t1: float):
        """Median SM MHz, active reasons and sample count between two perf_counter times."""
        inside = [(m, r) for (t, m, r) in list(self.samples) if t0 <= t <= t1]
        mask = 0
        for _, r in inside:
            mask |= r
        reasons = sorted(name for name, bit in self.REASONS.items() if mask & bit)
        return (statistics.median(m for m, _ in inside) if inside else None), reasons, len(inside)

    def stop(self):
        if not self.thread:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": "unavailable"}
        self._stop.set()
        self.thread.join(timeout=2)
        mhz, reasons, n = self.window(self.marks.get("begin", 0.0), self.marks.get("end", float("inf")))
        return {"sm_mhz": mhz, "sm_max_mhz": self.sm_max, "reasons": reasons, "samples": n,
                "source": "nvml polling during the timed region"}


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
def _cpu_operands(rows: int):
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16)
    a = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    return a, w


def cpu_gemm_sample(target_seconds: float):
    """Times the oracle's fp32 CPU matmul on the fixed row slab of the same GEMM (full K and N),
    repeated for about `target_seconds`; returns (TFLOP/s, threads, description)."""
    from oracle import oracle
    torch.set_num_threads(host_threads())
    threads = torch.get_num_threads()
    rows = REFERENCE_SAMPLE_ROWS
    a, w = _cpu_operands(rows)
    oracle.gemm_ref(a, w)  # warm-up (thread pool, page faults)
    best, spent, reps = None, 0.0, 0
    while spent < target_seconds or reps < 2:
        t0 = time.perf_counter()
        oracle.gemm_ref(a, w)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        spent += dt
        reps += 1
    tflops = 2.0 * rows * N * K / best / 1e12
    sample = (f"fp32 torch.matmul on CPU, {rows} of {M} rows x full K={K}, N={N} (bf16-rounded operands widened "
              f"to fp32), best of {reps} passes")
    return tflops, threads, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps, warmup = args.steps, args.warmup
    from oracle import oracle
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm takes every core
    # this process may run on, at every N
    torch.set_num_threads(host_threads())
    threads = torch.get_num_threads()
    rows = REFERENCE_SAMPLE_ROWS
    a, w = _cpu_operands(rows)
    for _ in range(max(1, warmup)):
        oracle.gemm_ref(a, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.gemm_ref(a, w)
    dt = time.perf_counter() - t0
    value = 2.0 * rows * N * K * steps / dt / 1e12
    sample = (f"each step: fp32 torch.matmul on CPU of {rows} of {M} rows x full K={K}, N={N} "
              "(bf16-rounded operands widened to fp32)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "sample_rows": rows},
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
        fn = lambda: fmha.fmha_fwd(q, k, v, causal=True, out=o, variant=args.variant)
        work, unit = 4.0 * 32 * 4096 * 4096 * 128 * 0.5 / 1e12, "TFLOP/s"
    elif case == "fmha_d64":
        # bf16, B=2 of the 8, 32 heads, s=2048, d=64, full: 50 MB per tensor
        q = inputs.device_randn16((2, 32, 2048, 64), 1, 1.0, torch.bfloat16, dev)
        k, v = torch.randn_like(q), torch.randn_like(q)
        o = torch.empty_like(q)
        fn = lambda: fmha.fmha_fwd(q, k, v, causal=False, out=o, variant=args.variant)
        work, unit = 4.0 * 2 * 32 * 2048 * 2048 * 64 / 1e12, "TFLOP/s"
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
class _Env:
    """Process-wide state of one rank of the GPU arm."""

    def __init__(self, args):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                             "use --impl reference for the CPU arm")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.distributed = self.world > 1
        if self.distributed:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.steps, self.warmup = args.steps, max(args.warmup, 3)
        self.peaks = measured_peaks()

    def barrier(self):
        if self.distributed:
            self.dist.barrier()

    def max_over_ranks(self, seconds: float) -> float:
        if not self.distributed:
            return seconds
        t = torch.tensor([seconds], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, flag: bool) -> bool:
        if not self.distributed:
            return bool(flag)
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())


def _e2e_gemm(env, a, w_mine, n_cols, steps):
    """The reference-facing op with HOST operands: every step copies A and this rank's weight columns
    in from pinned memory, calls fine_gemm, and copies this rank's columns of C back.  Pipelined over
    three buffer sets and copy-in / compute / copy-out streams, so the PCIe directions and the GPU
    overlap; every step still moves all of its inputs and its whole result."""
    import gemm_unified
    a_h = a.cpu().pin_memory()
    w_h = w_mine.contiguous().cpu().pin_memory()
    nbuf = 3
    a_d = [torch.empty_like(a) for _ in range(nbuf)]
    w_d = [torch.empty((K, n_cols), dtype=torch.bfloat16, device=env.dev) for _ in range(nbuf)]
    c_hs = [torch.empty((M, n_cols), dtype=torch.bfloat16).pin_memory() for _ in range(nbuf)]
    st_in, st_run, st_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def run(nsteps):
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

    run(4)  # warm-up
    env.barrier()
    secs = env.max_over_ranks(run(steps))
    env.barrier()
    h2d = a_h.numel() * 2 + w_h.numel() * 2
    d2h = c_hs[0].numel() * 2
    return secs, h2d, d2h


def _extra_fmha_prefill(env, extra):
    """Causal prefill configuration (fp16, B=1, 32/8 heads, s=4096, d=128): device-resident rate with
    its roofline; at N=1 also the end-to-end rate through fine_fmha with host tensors and the CPU
    baseline (the reference test's fp32 `torch_attn` on a slice of the heads)."""
    from b200k import fmha, inputs
    import fmha_unified
    dev, world = env.dev, env.world
    q, k, v = inputs.fmha_c3(dev)
    o = torch.empty_like(q)
    fsteps = max(env.steps, 50)
    fsecs = env.max_over_ranks(time_cuda(lambda: fmha.fmha_fwd(q, k, v, causal=True, out=o), fsteps, env.warmup,
                                         env.barrier, warm_seconds=0.03))
    fflops = 4.0 * 1 * 32 * 4096 * 4096 * 128 * 0.5
    tf = world * fflops * fsteps / fsecs / 1e12
    rec = {
        "workload": "causal_fmha_fp16_B1_H32_8_S4096_D128", "value": tf, "unit": "TFLOP/s",
        "ms": fsecs / fsteps * 1e3, "flops_convention": "executed (causal half counted once)",
        "reference_convention_tflops": 2 * tf,
        "scaling": "one replica of the configuration per GPU" if world > 1 else "single GPU",
        "roofline": {"bound": "tensor", "achieved": tf / world, "peak": env.peaks["tflops"], "unit": "TFLOP/s",
                     "frac": tf / world / env.peaks["tflops"], "frac_of_nominal_2250": tf / world / 2250.0,
                     "traffic": None}}
    extra["fmha_prefill"] = rec
    if world > 1:
        return
    # end to end: pinned host q, k, v in, o out, through the reference-facing wrapper
    q_h, k_h, v_h = (t.cpu().pin_memory() for t in (q, k, v))
    o_h = torch.empty(q.shape, dtype=q.dtype).pin_memory()

    def e2e_step():
        qd = q_h.to(dev, non_blocking=True)
        kd = k_h.to(dev, non_blocking=True)
        vd = v_h.to(dev, non_blocking=True)
        o_h.copy_(fmha_unified.ops.fine_fmha(qd, kd, vd, True, False, 5), non_blocking=True)

    esteps = max(10, min(env.steps, 30))
    esecs = time_cuda(e2e_step, esteps, 3)
    rec["e2e"] = {"value": fflops * esteps / esecs / 1e12, "unit": "TFLOP/s", "ms": esecs / esteps * 1e3,
                  "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * 2,
                  "d2h_bytes_per_step": o_h.numel() * 2,
                  "api": "fmha_unified.ops.fine_fmha(q, k, v, True, False, 5)"}
    if not env.no_cpu:
        from oracle import oracle
        torch.set_num_threads(host_threads())
        heads = 8  # two of the eight KV groups: a quarter of the configuration
        qc, kc, vc = q_h[:, :heads].float(), k_h[:, :heads // 4].float(), v_h[:, :heads // 4].float()
        oracle.torch_attn_ref(qc, kc, vc, True)
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            oracle.torch_attn_ref(qc, kc, vc, True)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        rec["cpu_baseline"] = {
            "value": fflops * heads / 32 / best / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "port", "extrapolated": True,
            "sample": f"fp32 repeat_kv + scaled_dot_product_attention on CPU (the reference test's torch_attn), "
                      f"{heads} of 32 query heads, all 4096 rows; rate of the slice, best of 3"}


def _extra_decode(env, extra):
    """Split-KV decode configuration (fp16, B=64, s_q=1, 32/8 heads, d=128, KV lengths uniform in
    [512, 32768]): device-resident GB/s with its roofline; at N=1 also end to end through
    fine_fmha_decode_varlen with host tensors (on 16 of the 64 sequences: the padded K and V of the
    whole batch are 8 GiB) and the CPU baseline (fp32 torch_attn on 4 sequences)."""
    from b200k import fmha, inputs
    import fmha_unified
    dev, world = env.dev, env.world
    B, Hq, Hkv, Skv, D = 64, 32, 8, 32768, 128
    lens_host = inputs.decode_lens(B)
    lens = lens_host.to(dev)
    qd = inputs.device_randn16((B, Hq, 1, D), 7, 1.0, torch.float16, dev)
    kd = inputs.device_randn16((B, Hkv, Skv, D), 8, 1.0, torch.float16, dev)
    vd = inputs.device_randn16((B, Hkv, Skv, D), 9, 1.0, torch.float16, dev)
    od = torch.empty_like(qd)
    ws = fmha.decode_workspace(B, Hq, Hkv, 1, Skv, D, 0, dev)
    dsteps = max(env.steps, 10)
    dsecs = env.max_over_ranks(time_cuda(
        lambda: fmha.fmha_decode(qd, kd, vd, kv_lens=lens, out=od, workspace=ws), dsteps, env.warmup, env.barrier,
        warm_seconds=0.03))
    dbytes = float(lens_host.sum().item()) * Hkv * D * 2 * 2 + 2.0 * B * Hq * D * 2
    gbs = world * dbytes * dsteps / dsecs / 1e9
    rec = {
        "workload": "decode_fp16_B64_Sq1_H32_8_D128_kvlen_U512_32768", "value": gbs, "unit": "GB/s",
        "ms": dsecs / dsteps * 1e3, "bytes": "valid K+V once, q and o once",
        "scaling": "one replica of the configuration per GPU" if world > 1 else "single GPU",
        "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": env.peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / world / env.peaks["hbm_gbs"], "frac_of_nominal_8000": gbs / world / 8000.0,
                     "traffic": None}}
    extra["decode_splitkv"] = rec
    if world > 1:
        return
    Be = 16
    q_h = qd[:Be].cpu().pin_memory()
    k_h, v_h = kd[:Be].cpu().pin_memory(), vd[:Be].cpu().pin_memory()
    l_h = lens_host[:Be].clone().pin_memory()
    o_h = torch.empty(q_h.shape, dtype=q_h.dtype).pin_memory()
    del kd, vd
    torch.cuda.empty_cache()

    def e2e_step():
        qx = q_h.to(dev, non_blocking=True)
        kx = k_h.to(dev, non_blocking=True)
        vx = v_h.to(dev, non_blocking=True)
        lx = l_h.to(dev, non_blocking=True)
        o_h.copy_(fmha_unified.ops.fine_fmha_decode_varlen(qx, kx, vx, lx), non_blocking=True)

    esecs = time_cuda(e2e_step, 4, 2)
    ebytes = float(lens_host[:Be].sum().item()) * Hkv * D * 4 + 2.0 * Be * Hq * D * 2
    rec["e2e"] = {"value": ebytes * 4 / esecs / 1e9, "unit": "GB/s", "ms": esecs / 4 * 1e3,
                  "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * 2 + l_h.numel() * 4,
                  "d2h_bytes_per_step": o_h.numel() * 2,
                  "api": "fmha_unified.ops.fine_fmha_decode_varlen(q, k, v, kv_lens)",
                  "sample": f"{Be} of the 64 sequences; the whole padded K and V of those sequences are copied in "
                            "every step, the rate counts their valid bytes only"}
    if not env.no_cpu:
        from oracle import oracle
        torch.set_num_threads(host_threads())
        nseq = 4
        seqs = []
        for b in range(nseq):
            n = int(lens_host[b])
            seqs.append((q_h[b:b + 1].float(), k_h[b:b + 1, :, :n].float(), v_h[b:b + 1, :, :n].float()))
        for (qc, kc, vc) in seqs:
            oracle.torch_attn_ref(qc, kc, vc, False)
        t0 = time.perf_counter()
        for (qc, kc, vc) in seqs:
            oracle.torch_attn_ref(qc, kc, vc, False)
        dt = time.perf_counter() - t0
        cbytes = float(lens_host[:nseq].sum().item()) * Hkv * D * 4 + 2.0 * nseq * Hq * D * 2
        rec["cpu_baseline"] = {
            "value": cbytes / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "extrapolated": True,
            "sample": f"fp32 repeat_kv + scaled_dot_product_attention on CPU (the reference test's torch_attn), "
                      f"{nseq} of the 64 sequences, one call per sequence over its valid keys (fp32 copies made "
                      "outside the timed region); rate in the same 16-bit algorithmic bytes"}


def _extra_skinny(env, extra):
    """Skinny GEMM paired with the decode configuration: M=64 tokens against the 4096x11008 weight,
    8 weight copies rotated so that the weight is streamed from HBM, not from L2."""
    from b200k import gemm, inputs
    dev, world = env.dev, env.world
    Ms, Ks, Ns = 64, 4096, 11008
    xs = inputs.device_randn16((Ms, Ks), 11, 1.0, torch.bfloat16, dev)
    wts = [inputs.device_randn16((Ks, Ns), 20 + t, 0.02, torch.bfloat16, dev) for t in range(8)]
    cs = torch.empty((Ms, Ns), dtype=torch.bfloat16, device=dev)
    turn = [0]

    def skinny_step():
        turn[0] = (turn[0] + 1) % len(wts)
        gemm.gemm(xs, wts[turn[0]], out=cs)

    ssteps = max(env.steps, 200)
    ssecs = env.max_over_ranks(time_cuda(skinny_step, ssteps, env.warmup, env.barrier, warm_seconds=0.03))
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
    gsecs = env.max_over_ranks(time_cuda(graph.replay, gsteps, 3, env.barrier)) / len(wts)
    ggbs = world * sbytes * gsteps / gsecs / 1e9
    extra["skinny_gemm"] = {
        "workload": "gemm_bf16_M64_K4096_N11008", "value": ggbs, "unit": "GB/s", "ms": gsecs / gsteps * 1e3,
        "note": "launches replayed from a CUDA graph, weights rotated through 8 copies (HBM-resident, not L2)",
        "per_call_from_python": {"value": sgbs, "unit": "GB/s", "ms": ssecs / ssteps * 1e3,
                                 "note": "one launch per call through the binding, host overhead inside"},
        "roofline": {"bound": "hbm", "achieved": ggbs / world, "peak": env.peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": ggbs / world / env.peaks["hbm_gbs"], "traffic": 94146304}}
    del graph


def _extra_host_path(env, extra):
    """The smallest configuration (fp16 1024^3, 64 tiles, a few microseconds of device time) through
    the reference-facing op, one call at a time: what a call costs on the host, next to torch.matmul
    (cuBLAS through torch's own dispatcher) on the same operands."""
    from b200k import inputs
    import gemm_unified
    a1, b1 = inputs.gemm_c1(env.dev)
    n = 2000
    rec = {"workload": "gemm_fp16_1024x1024x1024 (one call at a time)", "binding": gemm_unified._C.BINDING}
    for name, fn in (("fine_gemm", lambda: gemm_unified.ops.fine_gemm(a1, b1, 12)),
                     ("torch_matmul", lambda: torch.matmul(a1, b1))):
        secs = min(time_cuda(fn, n, 20) for _ in range(3))
        rec[name] = {"us_per_call": secs / n * 1e6, "tflops": 2.0 * 1024 ** 3 * n / secs / 1e12}
    extra["host_path"] = rec


def _extra_sustained(env, extra, a, w, c, sampler):
    """The headline GEMM under sustained load: about 2 s of launches in eight chunks alternating with
    torch.matmul (cuBLAS) on the same operands, so both run at the clocks the 1 kW power cap allows;
    TFLOP/s, the median SM clock of each arm's chunks, and TFLOP/s scaled to the maximum clock."""
    from b200k import gemm
    c2 = torch.empty_like(c)
    arms = {"library": lambda: gemm.gemm(a, w, out=c), "torch_matmul": lambda: torch.matmul(a, w, out=c2)}
    chunk = 500  # launches per chunk: about 0.25 s
    warm_for(arms["library"], 0.3)
    total = {k: 0.0 for k in arms}
    spans = {k: [] for k in arms}
    for _ in range(4):
        for name, fn in arms.items():
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            total[name] += time_cuda(fn, chunk, 0)
            spans[name].append((t0, time.perf_counter()))
    rec = {"workload": WORKLOAD, "launches_per_arm": 4 * chunk,
           "method": "4 chunks of 500 launches per arm, the arms alternating; clocks sampled through NVML"}
    for name in arms:
        tf = FLOPS_PER_STEP * 4 * chunk / total[name] / 1e12
        mhz = [m for (t0, t1) in spans[name] for m in [sampler.window(t0, t1)[0]] if m]
        reasons = sorted({r for (t0, t1) in spans[name] for r in sampler.window(t0, t1)[1]})
        med = statistics.median(mhz) if mhz else None
        rec[name] = {"tflops": tf, "seconds": total[name], "sm_mhz_median": med, "reasons": reasons,
                     "tflops_at_max_clock": tf * sampler.sm_max / med if med and sampler.sm_max else None}
    if env.peaks.get("tflops_sustained"):
        rec["frac_of_measured_sustained_peak"] = rec["library"]["tflops"] / env.peaks["tflops_sustained"]
        rec["measured_sustained_peak"] = env.peaks["tflops_sustained"]
    extra["gemm_sustained"] = rec


def _extra_sharded_attention(env, extra):
    """Strong scaling of the attention paths: a FIXED problem sharded over the ranks.
    prefill: bf16, B=8, 32 heads (MHA), s=2048, d=128, causal, (batch, head) pairs dealt to the ranks;
    decode: the 64-sequence batch, sequences balanced by total KV length.  No collective: the
    output stays sharded; the time is the slowest rank's."""
    from b200k import fmha, inputs, shard
    dev, world, rank = env.dev, env.world, env.rank
    Bp, Hp, Sp, Dp = 8, 32, 2048, 128
    mine = shard.head_shards(Bp, Hp, Hp, world)[rank]
    parts = []
    for (bb, h0, nh) in mine:
        qs = inputs.device_randn16((1, nh, Sp, Dp), 300 + bb * Hp + h0, 1.0, torch.bfloat16, dev)
        parts.append((qs, torch.randn_like(qs), torch.randn_like(qs), torch.empty_like(qs)))

    def prefill_shard():
        for (q_, k_, v_, o_) in parts:
            fmha.fmha_fwd(q_, k_, v_, causal=True, out=o_)

    psteps = max(env.steps, 10)
    psecs = env.max_over_ranks(time_cuda(prefill_shard, psteps, env.warmup, env.barrier))
    pflops = 4.0 * Bp * Hp * Sp * Sp * Dp * 0.5
    extra["fmha_prefill_sharded"] = {
        "workload": "causal_fmha_bf16_B8_H32_S2048_D128 over all ranks ((batch, head) shards)",
        "value": pflops * psteps / psecs / 1e12, "unit": "TFLOP/s", "ms": psecs / psteps * 1e3,
        "scaling": "strong", "launches_per_rank": len(parts)}
    # bit-exactness of a shard against the same slice of an unsharded launch, computed here
    q_, k_, v_, o_ = parts[0]
    nh = q_.size(1)
    pad = torch.randn((1, nh + 3, Sp, Dp), dtype=torch.bfloat16, device=dev)
    qf, kf, vf = (torch.cat((pad[:, :3], t), dim=1) for t in (q_, k_, v_))
    whole = fmha.fmha_fwd(qf, kf, vf, causal=True)
    attention_exact = torch.equal(whole[:, 3:], fmha.fmha_fwd(q_, k_, v_, causal=True))
    del parts, pad, qf, kf, vf, whole
    Bd, Hqd, Hkvd, Skvd, Dd = 64, 32, 8, 32768, 128
    all_lens = inputs.decode_lens(Bd)
    idx = shard.balance_sequences(all_lens.tolist(), world)[rank]
    nb_ = len(idx)
    lens_r = all_lens[idx].to(dev)
    qd = inputs.device_randn16((nb_, Hqd, 1, Dd), 7, 1.0, torch.float16, dev)
    kd = inputs.device_randn16((nb_, Hkvd, Skvd, Dd), 8, 1.0, torch.float16, dev)
    vd = inputs.device_randn16((nb_, Hkvd, Skvd, Dd), 9, 1.0, torch.float16, dev)
    od = torch.empty_like(qd)
    wsd = fmha.decode_workspace(nb_, Hqd, Hkvd, 1, Skvd, Dd, 0, dev)
    dsteps2 = max(env.steps, 10)
    dsecs2 = env.max_over_ranks(time_cuda(
        lambda: fmha.fmha_decode(qd, kd, vd, kv_lens=lens_r, out=od, workspace=wsd), dsteps2, env.warmup,
        env.barrier))
    dbytes2 = float(all_lens.sum().item()) * Hkvd * Dd * 4 + 2.0 * Bd * Hqd * Dd * 2
    extra["decode_sharded"] = {
        "workload": "the 64-sequence decode batch over all ranks (sequences balanced by KV length)",
        "value": dbytes2 * dsteps2 / dsecs2 / 1e9, "unit": "GB/s", "ms": dsecs2 / dsteps2 * 1e3,
        "scaling": "strong", "sequences_this_rank": nb_}
    # a sequence decoded alone equals its row of the batched launch (same split count)
    splits = 4
    one = fmha.fmha_decode(qd[:1], kd[:1], vd[:1], kv_lens=lens_r[:1], num_splits=splits)
    batch = fmha.fmha_decode(qd, kd, vd, kv_lens=lens_r, num_splits=splits)
    decode_exact = torch.equal(one, batch[:1])
    return attention_exact, decode_exact


def _extra_gemm_gather(env, extra, a, w):
    """N > 1: the one collective of the GEMM path, reassembling the column-sharded product on every
    rank: NCCL all-gather (as delivered, [ranks, M, slab]; and copied into row-major C) and fused into
    the GEMM epilogue (peer TMA stores + symmetric-memory barrier).  Also on a Llama-layer-sized
    activation (M = 65536 tokens), where the GEMM is long enough to hide the transfer."""
    from b200k import gemm, shard
    world, rank, dev = env.world, env.rank, env.dev
    slabs = shard.gemm_column_slabs(N, world)
    s0, e0 = slabs[rank]
    w_slab = w[:, s0:e0]
    gsteps = max(5, min(env.steps, 20))
    out_rm = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    t_slabs = env.max_over_ranks(time_cuda(
        lambda: shard.all_gather_slabs(gemm.gemm(a, w_slab), slabs), gsteps, 3, env.barrier))
    t_rowmajor = env.max_over_ranks(time_cuda(
        lambda: shard.all_gather_columns(gemm.gemm(a, w_slab), slabs, out=out_rm), gsteps, 3, env.barrier))
    fused = shard.FusedAllGatherGemm(M, N, torch.bfloat16, dev)
    t_fused = env.max_over_ranks(time_cuda(lambda: fused(a, w_slab), gsteps, 3, env.barrier))
    ingress = (world - 1) / world * M * N * 2  # bytes every GPU must receive
    link = 770e9                               # measured peer copy bandwidth per direction on this pool
    rec = {
        "workload": f"C[{M},{N}] = A . W with W column-sharded over {world} GPUs, full C on every rank",
        "nccl_slabs_ms": t_slabs / gsteps * 1e3, "nccl_rowmajor_ms": t_rowmajor / gsteps * 1e3,
        "fused_epilogue_ms": t_fused / gsteps * 1e3,
        "tflops_fused": FLOPS_PER_STEP * gsteps / t_fused / 1e12,
        "link_roofline": {"bytes_in_per_gpu": ingress, "peak_gbs_per_direction": link / 1e9,
                          "floor_ms": ingress / link * 1e3, "frac": ingress / link / (t_fused / gsteps)},
        "note": "nccl_slabs = local slab GEMM + all_gather_into_tensor, C left as [ranks, M, slab]; nccl_rowmajor "
                "adds the copy into row-major C; fused = epilogue TMA stores into all ranks' symmetric buffers "
                "(two buffers alternating) + symmetric-memory barrier"}
    # bit-exactness of both gathers against a rank-local full GEMM
    full = gemm.gemm(a, w)
    exact = torch.equal(fused(a, w_slab), full) and torch.equal(
        shard.all_gather_columns(gemm.gemm(a, w_slab), slabs), full)
    rec["bitexact_vs_local_full_gemm"] = env.all_true(exact)
    del fused, out_rm, full
    torch.cuda.empty_cache()
    # Llama-layer-sized activation: 65536 tokens
    Mb = 65536
    try:
        ab = torch.empty((Mb, K), dtype=torch.bfloat16, device=dev).normal_(0.0, 1.0)
        fused_b = shard.FusedAllGatherGemm(Mb, N, torch.bfloat16, dev)
        bsteps = 5
        t_fb = env.max_over_ranks(time_cuda(lambda: fused_b(ab, w_slab), bsteps, 2, env.barrier))
        t_lb = env.max_over_ranks(time_cuda(lambda: gemm.gemm(ab, w_slab), bsteps, 2, env.barrier))
        rec["m65536"] = {"fused_epilogue_ms": t_fb / bsteps * 1e3, "slab_gemm_only_ms": t_lb / bsteps * 1e3,
                         "tflops_fused": 2.0 * Mb * N * K * bsteps / t_fb / 1e12,
                         "link_floor_ms": (world - 1) / world * Mb * N * 2 / link * 1e3}
        del fused_b, ab
    except Exception as exc:
        rec["m65536"] = {"error": repr(exc)[:200]}
    extra["gemm_allgather_strong"] = rec
    return exact


def run_ours(args):
    from b200k import _lib, gemm, inputs, shard
    env = _Env(args)
    env.no_cpu = bool(args.no_cpu_baseline)
    dev, world, rank = env.dev, env.world, env.rank
    steps, warmup = env.steps, env.warmup
    _lib.lib()  # fail loudly here if the extension is missing

    # ---- headline GEMM: the fixed 8192 x 4096 x 11008 product, rank r computing column slab r ----
    # every rank holds the same A and the same full weight (same seeds), and computes its own columns
    a = inputs.device_randn16((M, K), 100, 1.0, torch.bfloat16, dev)
    w = inputs.device_randn16((K, N), 200, 0.02, torch.bfloat16, dev)
    slabs = shard.gemm_column_slabs(N, world)
    s0, e0 = slabs[rank]
    w_mine = w[:, s0:e0]
    c = torch.empty((M, e0 - s0), dtype=torch.bfloat16, device=dev)

    def step():
        gemm.gemm(a, w_mine, out=c)

    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    secs = env.max_over_ranks(time_cuda(step, steps, warmup, env.barrier, sampler if rank == 0 else None))
    launches = _lib.launch_count() - launches0 - warmup
    clocks = sampler.stop() if rank == 0 else None
    code, detail = _lib.device_status()
    if code != 0:
        raise SystemExit(f"device status {code} detail {detail:#x} after the timed region")
    value = FLOPS_PER_STEP * steps / secs / 1e12          # whole job: the one GEMM, all ranks together
    slab_flops = 2.0 * M * (e0 - s0) * K
    kernel_tflops = slab_flops * steps / secs / 1e12      # rate of this rank's kernel
    extra = {}

    # sharded result == the same columns of a rank-local full GEMM, bit for bit
    c_full = gemm.gemm(a, w)
    gemm_exact = torch.equal(c, c_full[:, s0:e0])
    if world > 1:
        # per-GPU rate with every rank running the whole GEMM (independent replicas, no collective)
        cw = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        wsecs = env.max_over_ranks(time_cuda(lambda: gemm.gemm(a, w, out=cw), steps, warmup, env.barrier))
        extra["gemm_weak"] = {"workload": WORKLOAD + " on every rank (replicas)", "scaling": "weak",
                              "value": world * FLOPS_PER_STEP * steps / wsecs / 1e12, "unit": UNIT,
                              "ms": wsecs / steps * 1e3}
        del cw
    del c_full

    # ---- e2e: reference-facing op, host operands, copies inside the timed region ----
    e2e_steps = max(4, min(steps, 12))
    e2e_secs, h2d, d2h = _e2e_gemm(env, a, w_mine, e0 - s0, e2e_steps)
    e2e_value = FLOPS_PER_STEP * e2e_steps / e2e_secs / 1e12

    # ---- extras: each may fail without taking the headline down ----
    for fn in (_extra_fmha_prefill, _extra_decode, _extra_skinny):
        try:
            fn(env, extra)
        except Exception as exc:
            extra[fn.__name__ + "_error"] = repr(exc)[:300]
        torch.cuda.empty_cache()
    exact = {"gemm_column_slab": gemm_exact}
    try:
        exact["attention_head_shard"], exact["decode_sequence_shard"] = _extra_sharded_attention(env, extra)
    except Exception as exc:
        extra["sharded_error"] = repr(exc)[:300]
    torch.cuda.empty_cache()
    if world > 1:
        try:
            exact["gemm_gathers"] = _extra_gemm_gather(env, extra, a, w)
        except Exception as exc:
            extra["gemm_allgather_strong"] = {"error": repr(exc)[:300]}
    extra["sharded_bitexact"] = env.all_true(all(exact.values()))
    extra["sharded_bitexact_checks"] = sorted(exact)
    if world == 1:
        try:
            _extra_host_path(env, extra)
        except Exception as exc:
            extra["host_path"] = {"error": repr(exc)[:300]}
    if world == 1 and not args.no_sustained:
        try:
            sampler2 = ClockSampler(env.local_rank, period_s=0.005)
            sampler2.start()
            if sampler2.thread:
                cs = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
                _extra_sustained(env, extra, a, w, cs, sampler2)
                sampler2.stop()
        except Exception as exc:
            extra["gemm_sustained"] = {"error": repr(exc)[:300]}

    # ---- CPU baseline on rank 0 at N=1 ----
    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        tflops, threads, sample = cpu_gemm_sample(10.0)
        cpu = {"value": tflops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
               "sample_rows": REFERENCE_SAMPLE_ROWS}

    if rank == 0:
        e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * world if world > 1 else h2d,
               "d2h_bytes_per_step": M * N * 2,
               "api": "gemm_unified.ops.fine_gemm(a, b, 12)",
               "pipelining": "3 buffer sets, copy-in / compute / copy-out streams"}
        if world > 1:
            e2e["note"] = (f"every rank copies the replicated A and its own weight slab in and its own C columns "
                           f"out; the {world} ranks share the host's memory and PCIe paths, so this number does "
                           "not scale with the GPUs")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": secs / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": bench_config(world),
            "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": env.peaks["tflops"], "unit": "TFLOP/s",
                         "frac": kernel_tflops / env.peaks["tflops"],
                         "traffic": NCU_TRAFFIC_BYTES if world == 1 else None,
                         "algorithmic": "flops of this rank's launch (2*M*slab*K) / its CUDA-event duration",
                         "peak_source": env.peaks["source"] + " (burst cuBLAS bf16: the timed region is a few ms)",
                         "frac_of_nominal_2250": kernel_tflops / 2250.0},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if env.distributed:
        env.dist.barrier()
        env.dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 4 s sustained-load comparison")
    ap.add_argument("--profile-case", default=None,
                    choices=["gemm", "fmha", "fmha_d64", "decode", "decode_short", "skinny"],
                    help="run only this path on a capture-sized case (for ncu); prints its own short line")
    ap.add_argument("--variant", type=int, default=0, help="kernel variant for --profile-case gemm / fmha")
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
