"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations.  Tensors are drawn on the CPU in fp32 from
`torch.Generator().manual_seed(seed)`, rounded to the 16-bit dtype and only then
copied to the device, so a CPU checker and the GPU kernels see identical bits.

The reference's own harness draws unseeded `torch.randn` on the GPU
(kernels/gemm/test/perf.py:8-9, kernels/fmha/test/perf.py:45-47); the seeds
here make runs repeatable.  Weights "shaped like Llama-2-7B" are random
N(0, 0.02) matrices of those shapes; no checkpoint is involved.
"""
from __future__ import annotations

import torch

# (K, N) of the Llama-2-7B projections: attention out / q, gate|up, down, fused QKV
LLAMA7B_KN = [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 12288)]
LLM_M = [1, 16, 128, 2048, 8192]


def randn16(shape, seed: int, std: float = 1.0, dtype=torch.float16, device="cpu") -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(*shape, generator=g, dtype=torch.float32)
    if std != 1.0:
        t = t * std
    return t.to(dtype).to(device)


def gemm_c1(device="cpu"):
    """fp16 1024^3, A and B ~ N(0,1)*0.1, seed 0."""
    g = torch.Generator().manual_seed(0)
    a = (torch.randn(1024, 1024, generator=g) * 0.1).to(torch.float16)
    b = (torch.randn(1024, 1024, generator=g) * 0.1).to(torch.float16)
    return a.to(device), b.to(device)


def gemm_llm(M: int, K: int, N: int, dtype=torch.bfloat16, device="cpu", seed: int = 1):
    """Activations N(0,1) [M,K], weights N(0,0.02) [K,N]."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(K, N, generator=g) * 0.02).to(dtype)
    return a.to(device), w.to(device)


def fmha_inputs(B: int, Hq: int, Hkv: int, Sq: int, Skv: int, D: int, dtype=torch.float16, device="cpu",
                seed: int = 2, layout: str = "bhsd"):
    """q [B,Hq,Sq,D], k, v [B,Hkv,Skv,D] ~ N(0,1).  layout "bshd" returns the same
    values stored [B,S,H,D] and viewed as [B,H,S,D] (strided, no copy)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Sq, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Skv, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, Skv, D, generator=g).to(dtype)
    if layout == "bshd":
        q, k, v = (t.transpose(1, 2).contiguous().to(device).transpose(1, 2) for t in (q, k, v))
        return q, k, v
    return q.to(device), k.to(device), v.to(device)


def fmha_c3(device="cpu", layout="bhsd"):
    """Causal prefill: fp16, B=1, 32 query / 8 KV heads, s=4096, d=128, seed 2."""
    return fmha_inputs(1, 32, 8, 4096, 4096, 128, torch.float16, device, seed=2, layout=layout)


def decode_lens(B: int = 64, lo: int = 512, hi: int = 32768, seed: int = 4) -> torch.Tensor:
    """Per-sequence KV lengths, uniform integers in [lo, hi]."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (B,), generator=g, dtype=torch.int32)


def device_randn16(shape, seed: int, std: float = 1.0, dtype=torch.float16, device="cuda") -> torch.Tensor:
    """Large tensors for timed runs only (drawn on the device: values differ from
    the CPU stream, so these are never compared against a CPU checker)."""
    g = torch.Generator(device=device).manual_seed(seed)
    t = torch.empty(shape, dtype=dtype, device=device)
    t.normal_(0.0, std, generator=g)
    return t
