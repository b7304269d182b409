"""Tensor-level wrapper of b200k_gemm."""
from __future__ import annotations

import torch

from . import _lib

AUTO, ONE_CTA, TWO_CTA, SKINNY, ONE_CTA_N128, GENERIC, TWO_CTA_N128, ONE_CTA_N64 = 0, 1, 2, 3, 4, 5, 6, 7

_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _check_inputs(a: torch.Tensor, b: torch.Tensor) -> None:
    # same conditions, in the same order, as the reference launchers
    # (kernels/gemm/pkg/gemm_unified/csrc/auto/gemm_0.cu:25-31), plus bf16
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("a and b must be 2-D")
    if a.size(1) != b.size(0):
        raise RuntimeError(f"shape mismatch: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if a.dtype not in _DTYPES or b.dtype != a.dtype:
        raise RuntimeError(f"a and b must both be float16 or bfloat16, got {a.dtype} and {b.dtype}")
    if not a.is_cuda or not b.is_cuda:
        raise RuntimeError("a and b must be CUDA tensors")
    if a.device != b.device:
        raise RuntimeError("a and b must be on the same device")


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, variant: int = AUTO) -> torch.Tensor:
    """C = a @ b with fp32 accumulation on the sm_100a kernels; a [M,K], b [K,N] row-major."""
    _check_inputs(a, b)
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    M, K = a.shape
    N = b.size(1)
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    elif out.shape != (M, N) or out.dtype != a.dtype or out.device != a.device or out.stride(1) != 1:
        raise RuntimeError("out has the wrong shape, dtype, device or layout")
    if M == 0 or N == 0:
        return out
    if K == 0:
        return out.zero_()
    L = _lib.lib()
    dev_index = a.device.index
    if dev_index is not None and dev_index != torch.cuda.current_device():
        with _lib.on_device(a.device):
            return gemm(a, b, out=out, variant=variant)
    # no variant needs a workspace (split-K partials stay in shared memory), so none is allocated
    code = L.b200k_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                        a.stride(0), b.stride(0), out.stride(0), _DTYPES[a.dtype], variant,
                        None, 0, _lib.raw_stream(a.device))
    if code:
        _lib.check(code, "b200k_gemm")
    return out


EPI_ADD, EPI_SWIGLU = 1, 2


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[K,F] gate and up projection weights -> one [K,2F] weight with gate_j at column 2j and up_j
    at column 2j+1 (a one-time weight transform), the layout the SwiGLU epilogue expects."""
    K, F = w_gate.shape
    return torch.stack((w_gate, w_up), dim=2).reshape(K, 2 * F).contiguous()


def _fused(a, b, residual, epilogue, out):
    _check_inputs(a, b)
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    M, K = a.shape
    N = b.size(1)
    n_out = N // 2 if epilogue == EPI_SWIGLU else N
    if out is None:
        out = torch.empty((M, n_out), dtype=a.dtype, device=a.device)
    elif out.shape != (M, n_out) or out.dtype != a.dtype or out.stride(1) != 1:
        raise RuntimeError("out has the wrong shape, dtype or layout")
    if residual is not None:
        if residual.shape != (M, N) or residual.dtype != a.dtype or residual.device != a.device:
            raise RuntimeError("residual must be [M,N] with the operands' dtype and device")
        if residual.stride(1) != 1:
            residual = residual.contiguous()
    if M == 0 or N == 0:
        return out
    with _lib.on_device(a.device):
        code = _lib.lib().b200k_gemm_fused(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None,
            M, N, K, a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
            _DTYPES[a.dtype], epilogue, _lib.raw_stream(a.device))
    _lib.check(code, "b200k_gemm_fused")
    return out


def gemm_add(a: torch.Tensor, b: torch.Tensor, residual: torch.Tensor, out: torch.Tensor | None = None):
    """a @ b + residual with the add fused into the GEMM epilogue (fp32 before rounding)."""
    return _fused(a, b, residual, EPI_ADD, out)


def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor | None = None):
    """silu(a @ w_gate) * (a @ w_up) for w_gate_up = interleave_gate_up(w_gate, w_up), fused."""
    return _fused(a, w_gate_up, None, EPI_SWIGLU, out)
