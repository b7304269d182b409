"""Registers the reference's GEMM op schema and routes it to libb200k.so.

Same op names and signatures as the reference's TORCH_LIBRARY block
(kernels/gemm/pkg/gemm_unified/csrc/gemm_kernel.cu:9-27):
`gemm_unified::finegemm_{0..16}(Tensor a, Tensor b) -> Tensor`.  Indices 0..12
(every index the reference implements for NVIDIA) get a CUDA implementation;
13..16 stay declared only, as in the reference's NVIDIA build, so calling them
raises the dispatcher's "no kernel" error.

The reference's rungs differ in technique, not in contract; here an index
selects a variant of the sm_100a kernel family instead:
   0..7, 12  heuristic choice        8   CUDA-core kernel (no alignment rules)
   9         128x128 tiles, 1 CTA    10  128x256 tiles, 1 CTA
   11        256x256 tiles, CTA pair

The registration itself lives in C++ when the compiled binding has been built
(torch_shim/ops_shim.cpp, loaded here), otherwise in this module over ctypes; see b200k/_binding.py.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from b200k import _binding, gemm as _gemm  # noqa: E402

NUM_DECLARED = 17
VARIANT_OF_INDEX = {i: _gemm.AUTO for i in range(13)}
VARIANT_OF_INDEX.update({8: _gemm.GENERIC, 9: _gemm.ONE_CTA_N128, 10: _gemm.ONE_CTA, 11: _gemm.TWO_CTA})

BINDING = _binding.binding()  # "compiled": the C++ TORCH_LIBRARY blocks are loaded and nothing is defined here


def _make_impl(variant: int):
    def impl(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return _gemm.gemm(a, b, variant=variant)
    return impl


if BINDING == "ctypes":
    _library = torch.library.Library("gemm_unified", "DEF")
    for _i in range(NUM_DECLARED):
        _library.define(f"finegemm_{_i}(Tensor a, Tensor b) -> Tensor")
    for _i, _variant in VARIANT_OF_INDEX.items():
        _library.impl(f"finegemm_{_i}", _make_impl(_variant), "CUDA")
