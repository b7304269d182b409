import torch
from torch import Tensor

__all__ = ["fine_fmha", "fine_fmha_decode_varlen"]

_KERNELS = {}


def fine_fmha(q: Tensor, k: Tensor, v: Tensor, causal: bool, is_decode, kernel_index: int) -> Tensor:
    """Attention forward through `torch.ops.fmha_unified.finefmha_{kernel_index}`.

    Same signature and result as the reference's wrapper
    (kernels/fmha/pkg/fmha_unified/ops.py:8-29): q [B,Hq,S,d], k, v [B,Hkv,Skv,d],
    output [B,Hq,S,d].  The reference pads q, k, v along the sequence to a
    multiple of 64, copies them and slices the output (:15-29) because its kernels
    have no tail handling; these kernels clip ragged tiles themselves, so the
    tensors are passed as they are (no copy) with `decode_length = k.size(2)` (:18).
    """
    kernel = _KERNELS.get(kernel_index)
    if kernel is None:
        kernel = getattr(torch.ops.fmha_unified, f"finefmha_{int(kernel_index)}").default
        _KERNELS[kernel_index] = kernel
    return kernel(q, k, v, bool(causal), bool(is_decode), k.size(2))


def fine_fmha_decode_varlen(q: Tensor, k: Tensor, v: Tensor, kv_lens: Tensor) -> Tensor:
    """Decode attention over a padded KV batch with per-sequence valid lengths
    (int32 [B] on the device).  No counterpart in the reference, whose ops carry
    one scalar `decode_length` for the whole batch."""
    return torch.ops.fmha_unified.finefmha_decode_varlen.default(q, k, v, kv_lens)
