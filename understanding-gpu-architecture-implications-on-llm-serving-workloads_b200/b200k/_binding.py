"""Chooses how the reference's torch ops reach libb200k.so.

Two bindings register the same schemas (`gemm_unified::finegemm_{0..16}`,
`fmha_unified::finefmha_{0..7}`, `fmha_unified::finefmha_decode_varlen`):

  compiled  lib/libb200k_torch_ops.so (torch_shim/ops_shim.cpp): TORCH_LIBRARY / TORCH_LIBRARY_IMPL
            blocks in C++, as in the reference (kernels/gemm/pkg/gemm_unified/csrc/gemm_kernel.cu:9-27);
            a call goes dispatcher -> C++ -> C ABI.  Used when the library has been built.
  ctypes    the schemas defined from Python with torch.library and implemented by the
            tensor-level wrappers in b200k/gemm.py and b200k/fmha.py; a call goes
            dispatcher -> Python -> ctypes -> C ABI.  Used otherwise, or with B200K_BINDING=ctypes.

Both end in the same C-ABI entry points and kernels; only the host path differs.  One process uses
one binding for both namespaces (the compiled library defines both).
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

SHIM_PATH = Path(__file__).resolve().parent.parent / "lib" / "libb200k_torch_ops.so"

_choice = None


def binding() -> str:
    """"compiled" or "ctypes"; loads the compiled binding on first use when it is the choice."""
    global _choice
    if _choice is None:
        want = os.environ.get("B200K_BINDING", "").strip().lower()
        if want not in ("", "compiled", "ctypes"):
            raise RuntimeError(f"B200K_BINDING must be 'compiled' or 'ctypes', got {want!r}")
        if want == "compiled" and not SHIM_PATH.exists():
            raise RuntimeError(f"{SHIM_PATH} is missing: build it with build.py (B200K_BINDING=compiled)")
        if want != "ctypes" and SHIM_PATH.exists():
            torch.ops.load_library(str(SHIM_PATH))
            _choice = "compiled"
        else:
            _choice = "ctypes"
    return _choice
