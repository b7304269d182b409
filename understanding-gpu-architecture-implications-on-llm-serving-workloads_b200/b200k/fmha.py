"""Tensor-level wrappers of b200k_fmha_fwd and b200k_fmha_decode_splitkv."""
from __future__ import annotations

import math

import torch

from . import _lib

_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
# query rows per KV head (query heads of the group x Sq) one launch of the split-KV kernel takes
MAX_DECODE_ROWS = 16


def _check_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    # conditions of the reference launchers
    # (kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_4_nv.cu:397-417), plus bf16 and d = 64
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("q, k, v must be [batch, heads, seq, head_dim]")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError(f"q, k, v must all be float16 or bfloat16, got {q.dtype}, {k.dtype}, {v.dtype}")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("q, k, v must be CUDA tensors")
    if not (q.device == k.device == v.device):
        raise RuntimeError("q, k, v must be on the same device")
    B, Hq, Sq, D = q.shape
    if k.shape != v.shape or k.size(0) != B or k.size(3) != D:
        raise RuntimeError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if k.size(1) == 0 or Hq % k.size(1) != 0:
        raise RuntimeError("number of query heads must be a multiple of the number of KV heads")
    if D not in (64, 128):
        raise RuntimeError(f"head_dim must be 64 or 128, got {D}")


def _rows_contiguous(t: torch.Tensor) -> torch.Tensor:
    """The kernels need the head_dim axis contiguous and 16-byte aligned strides;
    anything else (rare) is copied once."""
    if t.stride(3) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
        return t.contiguous()
    return t


def fmha_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, kv_len: int | None = None,
             scale: float | None = None, out: torch.Tensor | None = None, variant: int = 0) -> torch.Tensor:
    """softmax(q k^T scale + mask) v; q [B,Hq,Sq,D], k, v [B,Hkv,Skv,D] (any batch/head/row strides)."""
    _check_qkv(q, k, v)
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.size(1), k.size(2)
    if kv_len is None:
        kv_len = Skv
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=q.dtype, device=q.device)
    if Sq == 0 or B == 0:
        return out
    if Skv == 0 or kv_len <= 0:
        return out.zero_()
    q, k, v = _rows_contiguous(q), _rows_contiguous(k), _rows_contiguous(v)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    L = _lib.lib()
    with _lib.on_device(q.device):
        code = L.b200k_fmha_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, Hkv, Sq, Skv, D,
                                _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out),
                                float(scale), int(bool(causal)), int(min(kv_len, Skv)), _DTYPES[q.dtype], int(variant),
                                _lib.raw_stream(q.device))
    _lib.check(code, "b200k_fmha_fwd")
    return out


def decode_workspace(B: int, Hq: int, Hkv: int, Sq: int, Skv: int, D: int, num_splits: int, device) -> torch.Tensor:
    n = _lib.lib().b200k_fmha_decode_workspace_bytes(B, Hq, Hkv, Sq, Skv, D, num_splits)
    return torch.empty(max(int(n), 16), dtype=torch.uint8, device=device)


def fmha_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_lens: torch.Tensor | None = None,
                num_splits: int = 0, scale: float | None = None, out: torch.Tensor | None = None,
                workspace: torch.Tensor | None = None, static_scratch: bool = False) -> torch.Tensor:
    """Split-KV attention for decode-shaped inputs (q [B,Hq,Sq,D] with small Sq, normally 1).
    kv_lens: int32 [B] on the device (valid keys of each sequence) or None for all of Skv.
    static_scratch: use the entry point that keeps its partials in the library's built-in scratch
    array instead of a workspace tensor, for callers that must not allocate device memory on this path
    (the first such call on a device looks the array's address up and belongs outside a stream capture;
    calls that overlap on one GPU race on the shared array)."""
    _check_qkv(q, k, v)
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.size(1), k.size(2)
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=q.dtype, device=q.device)
    if Sq == 0 or B == 0:
        return out
    if Skv == 0:
        return out.zero_()
    group = Hq // Hkv
    if group * Sq > MAX_DECODE_ROWS and Sq <= MAX_DECODE_ROWS:
        # More query rows share a KV head than the kernel's 16-row tile holds (MQA, wide GQA groups):
        # the query heads of every group are taken in slices that fit, each slice one launch over the
        # same K/V (q and o are a few KB per sequence; K/V are not copied).
        per = max(g for g in range(1, group + 1) if group % g == 0 and g * Sq <= MAX_DECODE_ROWS)
        q5, o5 = q.unflatten(1, (Hkv, group)), out.unflatten(1, (Hkv, group))
        for j in range(0, group, per):
            part = fmha_decode(q5[:, :, j:j + per].flatten(1, 2), k, v, kv_lens=kv_lens, num_splits=num_splits,
                               scale=scale, workspace=workspace, static_scratch=static_scratch)
            o5[:, :, j:j + per].copy_(part.unflatten(1, (Hkv, per)))
        return out
    q, k, v = _rows_contiguous(q), _rows_contiguous(k), _rows_contiguous(v)
    if kv_lens is not None:
        if kv_lens.dtype != torch.int32 or kv_lens.device != q.device or kv_lens.numel() != B:
            raise RuntimeError("kv_lens must be an int32 tensor with one entry per batch element on q's device")
        kv_lens = kv_lens.contiguous()
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    L = _lib.lib()
    with _lib.on_device(q.device):
        if static_scratch:
            code = L.b200k_fmha_decode_splitkv_static(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, Hkv, Sq, Skv, D,
                _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out), float(scale),
                kv_lens.data_ptr() if kv_lens is not None else None, int(num_splits), _DTYPES[q.dtype],
                _lib.raw_stream(q.device))
            _lib.check(code, "b200k_fmha_decode_splitkv_static")
            return out
        if workspace is None:
            workspace = decode_workspace(B, Hq, Hkv, Sq, Skv, D, num_splits, q.device)
        code = L.b200k_fmha_decode_splitkv(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, Hkv, Sq, Skv, D,
            _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out), float(scale),
            kv_lens.data_ptr() if kv_lens is not None else None, int(num_splits), _DTYPES[q.dtype],
            workspace.data_ptr(), workspace.numel(), _lib.raw_stream(q.device))
    _lib.check(code, "b200k_fmha_decode_splitkv")
    return out


def fmha_decode_paged(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                      kv_lens: torch.Tensor, num_splits: int = 0, scale: float | None = None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Decode attention over a paged cache: k_pages, v_pages [num_pages, Hkv, page_size, D] (page_size a
    multiple of 64), block_table int32 [B, max_blocks] (page of every logical block), kv_lens int32 [B]."""
    if q.dim() != 4 or k_pages.dim() != 4 or k_pages.shape != v_pages.shape:
        raise RuntimeError("q must be [B,Hq,Sq,D]; k_pages and v_pages [num_pages,Hkv,page_size,D]")
    if q.dtype not in _DTYPES or k_pages.dtype != q.dtype or v_pages.dtype != q.dtype:
        raise RuntimeError("q, k_pages, v_pages must all be float16 or bfloat16")
    B, Hq, Sq, D = q.shape
    num_pages, Hkv, page_size, Dk = k_pages.shape
    if Dk != D or block_table.dim() != 2 or block_table.size(0) != B or block_table.dtype != torch.int32:
        raise RuntimeError("block_table must be int32 [B, max_blocks] and head_dim must match")
    if kv_lens.dtype != torch.int32 or kv_lens.numel() != B:
        raise RuntimeError("kv_lens must be int32 [B]")
    if not all(t.is_cuda and t.device == q.device for t in (k_pages, v_pages, block_table, kv_lens)):
        raise RuntimeError("all tensors must be on q's CUDA device")
    q, k_pages, v_pages = _rows_contiguous(q), _rows_contiguous(k_pages), _rows_contiguous(v_pages)
    block_table, kv_lens = block_table.contiguous(), kv_lens.contiguous()
    max_blocks = block_table.size(1)
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=q.dtype, device=q.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    L = _lib.lib()
    with _lib.on_device(q.device):
        ws = decode_workspace(B, Hq, Hkv, Sq, max_blocks * page_size, D, num_splits, q.device)
        code = L.b200k_fmha_decode_paged(
            q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), B, Hq, Hkv, Sq, D, num_pages,
            page_size, _lib.strides3(q), _lib.strides3(k_pages), _lib.strides3(v_pages), _lib.strides3(out),
            float(scale), block_table.data_ptr(), max_blocks, kv_lens.data_ptr(), int(num_splits), _DTYPES[q.dtype],
            ws.data_ptr(), ws.numel(), _lib.raw_stream(q.device))
    _lib.check(code, "b200k_fmha_decode_paged")
    return out
