"""ctypes binding of libb200k.so (the C ABI declared in include/b200k.h).

There is no fallback: if the library is missing, or the device is not an
sm_100 GPU, every call raises.  The host side stays Python/PyTorch exactly as
in the reference (kernels/gemm/pkg/gemm_unified/ops.py:7-13 and
kernels/fmha/pkg/fmha_unified/ops.py:8-29 are Python wrappers over C++ ops);
torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p, POINTER
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent.parent
LIB_PATH = Path(os.environ.get("B200K_LIB", PKG_DIR / "lib" / "libb200k.so"))

F16, BF16 = 0, 1

# every symbol include/b200k.h declares, with its ctypes signature
_I64x3 = POINTER(c_int64)
SIGNATURES = {
    "b200k_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                           c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200k_gemm_scatter": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int64,
                                   c_int64, c_int64, c_int, c_void_p]),
    "b200k_gemm_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                 c_int64, c_int64, c_int, c_int, c_void_p]),
    "b200k_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200k_fmha_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                               _I64x3, _I64x3, _I64x3, _I64x3, c_float, c_int, c_int, c_int, c_int, c_void_p]),
    "b200k_fmha_decode_splitkv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_int, _I64x3, _I64x3, _I64x3, _I64x3, c_float, c_void_p,
                                          c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200k_fmha_decode_splitkv_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, _I64x3, _I64x3, _I64x3, _I64x3, c_float, c_void_p,
                                                 c_int, c_int, c_void_p]),
    "b200k_fmha_decode_static_scratch_bytes": (c_size_t, []),
    "b200k_fmha_decode_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int, _I64x3, _I64x3, _I64x3, _I64x3, c_float, c_void_p, c_int, c_void_p,
                                        c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200k_fmha_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200k_fmha_decode_auto_splits": (c_int, [c_int, c_int, c_int]),
    "b200k_strerror": (c_char_p, [c_int]),
    "b200k_device_status": (c_int, [POINTER(c_int), POINTER(c_int)]),
    "b200k_launch_count": (c_uint64, []),
    "b200k_device_supported": (c_int, []),
    "b200k_set_option": (c_int, [c_int, c_int]),
    "b200k_debug_wait_timeout": (c_int, [c_uint64, c_void_p]),
    "b200k_debug_smem_desc": (c_uint64, [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]),
    "b200k_debug_instr_desc": (ctypes.c_uint32, [c_int, c_int, c_int, c_int, c_int]),
}


class B200KError(RuntimeError):
    """A libb200k entry point returned a negative code."""

    def __init__(self, code: int, where: str):
        self.code = code
        super().__init__(f"{where}: {strerror(code)} (code {code})")


_lib = None


def lib() -> ctypes.CDLL:
    """Loads libb200k.so once; raises if it was not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python {PKG_DIR / 'build.py'}` "
                "(there is no CPU or eager fallback)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def strerror(code: int) -> str:
    return lib().b200k_strerror(code).decode()


def check(code: int, where: str) -> None:
    if code != 0:
        raise B200KError(code, where)


OPT_SKINNY_S, OPT_SKINNY_BN, OPT_DECODE_HEADS_PER_CTA, OPT_FMHA_PERSISTENT, OPT_FMHA_SPLIT_P, OPT_SKINNY_PAIR, OPT_PDL = 0, 1, 2, 3, 4, 5, 6


class option:
    """`with option(OPT_SKINNY_S, 4): ...` sets a tuning override of the library (b200k_set_option)
    for the block and restores the previous value afterwards."""

    def __init__(self, which: int, value: int):
        self.which, self.value = which, value

    def __enter__(self):
        self.before = lib().b200k_set_option(self.which, self.value)
        if self.before < 0:
            raise B200KError(self.before, "b200k_set_option")
        return self

    def __exit__(self, *exc):
        lib().b200k_set_option(self.which, self.before)
        return False


def launch_count() -> int:
    return int(lib().b200k_launch_count())


def device_status() -> tuple[int, int]:
    """(code, detail) of the current device's status word; synchronises."""
    code, detail = c_int(0), c_int(0)
    check(lib().b200k_device_status(ctypes.byref(code), ctypes.byref(detail)), "b200k_device_status")
    return code.value, detail.value


def raw_stream(device) -> int:
    """Handle of torch's current stream on `device` for the C ABI.  torch.cuda.current_stream() builds a
    Stream object on every call (about a third of a wrapper's host time on a 10 us kernel); the raw
    accessor returns the same handle directly."""
    import torch
    index = device.index if device.index is not None else torch.cuda.current_device()
    getter = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if getter is not None:
        return getter(index)
    return torch.cuda.current_stream(device).cuda_stream


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def on_device(device):
    """Context manager that makes `device` current for the C call; free when it already is."""
    import torch
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def strides3(t) -> ctypes.Array:
    """(batch, head, row) element strides of a [B, H, S, D] tensor as int64[3]."""
    s = t.stride()
    return (c_int64 * 3)(s[0], s[1], s[2])
