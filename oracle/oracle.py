"""CPU oracle for the GEMM and FMHA-forward paths.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference
arm import this module, and only as the checker or the timed CPU baseline.
The product path (libb200k.so) never routes through it.

What it restates
----------------
* GEMM: C[i,j] = sum_k a[i*K+k] * b[k*N+j], row-major operands
  (kernels/gemm/pkg/gemm_unified/csrc/auto/gemm_0.cu:12-20), evaluated as the
  fp32 `torch.matmul` on CPU that the headline tolerance is stated against
  (the reference's own check is `a @ b`, kernels/gemm/test/correct.py:9-16).
* FMHA forward: O = softmax(Q K^T * scale + mask) V with
    - layout Q,O [B,H_q,N_q,d], K,V [B,H_kv,N_kv,d]
      (kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_2_nv.cu:22-23),
    - GQA mapping kv_head = q_head / (H_q / H_kv) (fmha_2_nv.cu:36,42-45),
    - scale 1/sqrt(d) (fmha_2_nv.cu:310),
    - causal rule "q_idx < k_idx -> -inf", aligned to the top-left corner
      (fmha_2_nv.cu:177-180); with N_q != N_kv the library aligns the diagonal
      to the bottom-right corner, which is identical whenever N_q == N_kv,
    - keys at or beyond the valid length are masked.  The reference masks
      `k_idx > decode_length` (fmha_2_nv.cu:181), which leaves key index
      == decode_length unmasked; that off-by-one is not reproduced, the true
      length is used, as the fp32 formula the tolerance is stated against needs.
  `fmha_ref` is the closed formula (the reference test's own oracle `torch_attn`,
  kernels/fmha/test/correct.py:10-24); `fmha_ref_online` restates the blocked
  online-softmax recurrences of the kernels (fmha_2_nv.cu:173-208, final O/l at
  :283) in fp32 numpy, so tests can show the two agree.

Pinning
-------
The reference ships no golden vectors or known-answer files for these paths
(its correct.py scripts compare against torch on the GPU at run time, and the
FMHA one currently compares against raw QK^T, kernels/fmha/test/correct.py:52).
The oracle is pinned to the reference itself in two ways:
* tests/golden/: outputs of the reference's own oracle function, `torch_attn`
  IMPORTED from kernels/fmha/test/perf.py:10-24 (and `a @ b`,
  kernels/gemm/test/correct.py:9-16), generated in the build container with the
  reference's seeds and shapes by tests/golden/make_golden.py;
  tests/test_oracle_cpu.py holds the oracle to them on CPU;
* the reference's own CUDA rungs (finegemm_8 / _11, finefmha_2 / _4), compiled
  from the reference's sources by oracle/build_ref_ladder.py into oracle/_ref/
  and run in a child process by oracle/run_ref_check.py on the reference's
  check inputs (kernels/gemm/test/correct.py:5-16, kernels/fmha/test/correct.py:
  26-47): tests/test_reference_pin_gpu.py requires oracle <-> reference within
  the reference's tolerances and library <-> oracle within the stated ones on
  the same tensors.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# --------------------------------------------------------------------------- GEMM
def gemm_ref(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32 C = A.B on CPU from the (already 16-bit rounded) inputs."""
    return a.detach().cpu().float() @ b.detach().cpu().float()


def gemm_ref_loops(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """The reference's index arithmetic spelled out (auto/gemm_0.cu:12-20); float64
    accumulation, small cases only."""
    M, K = a.shape
    N = b.shape[1]
    af = a.astype(np.float64).reshape(-1)
    bf = b.astype(np.float64).reshape(-1)
    c = np.zeros(M * N, dtype=np.float64)
    for i in range(M):
        for j in range(N):
            acc = 0.0
            for k in range(K):
                acc += af[i * K + k] * bf[k * N + j]
            c[i * N + j] = acc
    return c.reshape(M, N)


# --------------------------------------------------------------------------- FMHA
def _kv_len_vector(kv_lens, B: int, n_kv: int) -> torch.Tensor:
    if kv_lens is None:
        return torch.full((B,), n_kv, dtype=torch.int64)
    if isinstance(kv_lens, int):
        return torch.full((B,), kv_lens, dtype=torch.int64)
    return torch.as_tensor(kv_lens).detach().cpu().to(torch.int64)


def fmha_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, kv_lens=None,
             scale: float | None = None) -> torch.Tensor:
    """fp32 softmax(Q K^T scale + mask) V on CPU.  q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D]."""
    q = q.detach().cpu().float()
    k = k.detach().cpu().float()
    v = v.detach().cpu().float()
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    assert Hq % Hkv == 0
    group = Hq // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    lens = _kv_len_vector(kv_lens, B, Skv)
    out = torch.empty_like(q)
    kidx = torch.arange(Skv)
    qidx = torch.arange(Sq)
    for b in range(B):
        n = int(lens[b])
        mask = (kidx[None, :] >= n)  # [1, Skv]
        if causal:
            # key j visible to query i when j <= i + (n - Sq): bottom-right aligned
            # to the valid length; equals `q_idx < k_idx -> masked` when Sq == n.
            mask = mask | (kidx[None, :] > (qidx[:, None] + (n - Sq)))
        for h in range(Hq):
            kk = torch.nan_to_num(k[b, h // group], nan=0.0) if n < Skv else k[b, h // group]
            vv = torch.nan_to_num(v[b, h // group], nan=0.0) if n < Skv else v[b, h // group]
            s = (q[b, h] @ kk.T) * scale
            s = s.masked_fill(mask, float("-inf"))
            p = torch.softmax(s, dim=-1)
            p = torch.nan_to_num(p, nan=0.0)  # rows with every key masked give 0
            out[b, h] = p @ vv
    return out


def torch_attn_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool) -> torch.Tensor:
    """The reference test scripts' own oracle as they compute it (kernels/fmha/test/perf.py:10-24,
    kernels/fmha/test/correct.py:10-24): every KV head repeated over its group of query heads
    (expand + reshape) and torch's scaled_dot_product_attention.  The group size is taken from the
    shapes (the scripts hard-code 4).  This is the function the CPU baseline of the attention paths
    times; `fmha_ref` is the same math with valid lengths and the bottom-right diagonal added."""
    if q.size(1) != k.size(1):
        n_rep = q.size(1) // k.size(1)
        b, h, s, d = k.shape
        k = k[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)
        v = v[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=is_causal)


def fmha_ref_online(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool = False, kv_len: int | None = None,
                    block: int = 64) -> np.ndarray:
    """Blocked online-softmax recurrences of the reference kernels in fp32 numpy
    (fmha_2_nv.cu:173-208,283): per key block j: m_new = max(m, rowmax(S_j));
    P = exp(S_j - m_new); l = exp(m - m_new) l + rowsum(P); O = exp(m - m_new) O + P V_j;
    finally O / l.  q [Hq,Sq,D], k/v [Hkv,Skv,D] for one batch entry."""
    q = q.astype(np.float32)
    k = k.astype(np.float32)
    v = v.astype(np.float32)
    Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[0], k.shape[1]
    group = Hq // Hkv
    n = Skv if kv_len is None else kv_len
    scale = np.float32(1.0 / math.sqrt(D))
    out = np.zeros_like(q)
    for h in range(Hq):
        kk, vv = k[h // group], v[h // group]
        m = np.full((Sq,), -np.inf, dtype=np.float32)
        l = np.zeros((Sq,), dtype=np.float32)
        o = np.zeros((Sq, D), dtype=np.float32)
        for j0 in range(0, n, block):
            j1 = min(j0 + block, n)
            s = (q[h] @ kk[j0:j1].T) * scale
            if causal:
                qi = np.arange(Sq)[:, None] + (n - Sq)
                kj = np.arange(j0, j1)[None, :]
                s = np.where(kj > qi, -np.inf, s)
            m_new = np.maximum(m, s.max(axis=1))
            safe = np.where(np.isinf(m_new), 0.0, m_new)
            p = np.exp(s - safe[:, None])
            alpha = np.exp(np.where(np.isinf(m), -np.inf, m - safe))
            l = alpha * l + p.sum(axis=1)
            o = alpha[:, None] * o + p @ vv[j0:j1]
            m = m_new
        out[h] = np.where(l[:, None] > 0, o / np.maximum(l, 1e-38)[:, None], 0.0)
    return out


# --------------------------------------------------------------------------- metrics
def rel_frobenius(x: torch.Tensor, ref: torch.Tensor) -> float:
    """||x - ref||_F / ||ref||_F in float64."""
    x = x.detach().cpu().double()
    ref = ref.detach().cpu().double()
    den = float(torch.linalg.norm(ref))
    num = float(torch.linalg.norm(x - ref))
    return num / den if den > 0 else num


def max_abs(x: torch.Tensor, ref: torch.Tensor) -> float:
    return float((x.detach().cpu().double() - ref.detach().cpu().double()).abs().max())


def bf16_ulp(ref: torch.Tensor) -> torch.Tensor:
    """Spacing of bfloat16 (8 significant bits) at |ref|, element-wise, in float64."""
    mag = ref.detach().cpu().double().abs().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(mag)) - 7)


def fmha_within_tolerance(o: torch.Tensor, ref: torch.Tensor, extra: float = 0.0,
                          absref: torch.Tensor | None = None) -> tuple[bool, float]:
    """The attention bar, returned as (ok, worst max-abs error).

    fp16 output: max-abs <= FMHA_MAX_ABS_TOL against the fp32 formula, as stated.
    bf16 output: a bf16 number cannot sit within 2e-3 of an fp32 value above ~0.5 (its spacing
    there is 2^-8 and up), and the probabilities P enter the second product as bf16 (8 significant
    bits, relative rounding error up to 2^-9 each).  So the unavoidable part is stated separately from
    the kernel's own error, three ways:
      * overall, against the unrounded formula: max-abs <= FMHA_MAX_ABS_TOL + 2^-8 max|ref|;
      * on average: relative Frobenius error <= 3e-3 (output rounding alone gives about 1.6e-3; a
        systematic 2^-8 error anywhere in the arithmetic would give 4e-3 or more);
      * per element, when `absref` = softmax(QK^T) |V| is given (the formula evaluated on |V|, which
        bounds how far rounding P can move each output): |o - bf16(ref)| <= FMHA_MAX_ABS_TOL + one bf16
        spacing at ref + 2^-8 absref, so an error cannot hide behind the largest output of the tensor."""
    o64, r64 = o.detach().cpu().double(), ref.detach().cpu().double()
    err = float((o64 - r64).abs().max())
    if o.dtype != torch.bfloat16:
        return err <= FMHA_MAX_ABS_TOL + extra, err
    ok = err <= FMHA_MAX_ABS_TOL + extra + float(r64.abs().max()) * 2.0 ** -8
    den = float(torch.linalg.norm(r64))
    ok = ok and (den == 0.0 or float(torch.linalg.norm(o64 - r64)) / den <= 3e-3)
    if absref is not None:
        rounded = ref.detach().cpu().float().to(torch.bfloat16).double()
        bound = FMHA_MAX_ABS_TOL + extra + bf16_ulp(ref) + absref.detach().cpu().double().abs() * 2.0 ** -8
        ok = ok and bool(((o64 - rounded).abs() <= bound).all())
    return ok, err


GEMM_REL_FRO_TOL = 1e-2   # stated tolerance: relative Frobenius error vs fp32 matmul
FMHA_MAX_ABS_TOL = 2e-3   # stated tolerance: max-abs vs fp32 softmax(QK^T scale)V
