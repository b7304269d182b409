import torch
from torch import Tensor

__all__ = ["fine_gemm"]

_KERNELS = {}


def fine_gemm(a: Tensor, b: Tensor, kernel_index: int) -> Tensor:
    """C = a @ b through `torch.ops.gemm_unified.finegemm_{kernel_index}`.

    Same signature as the reference's wrapper
    (kernels/gemm/pkg/gemm_unified/ops.py:7-13); the op lookup is cached
    instead of going through `exec` on every call.
    """
    kernel = _KERNELS.get(kernel_index)
    if kernel is None:
        kernel = getattr(torch.ops.gemm_unified, f"finegemm_{int(kernel_index)}").default
        _KERNELS[kernel_index] = kernel
    return kernel(a, b)
