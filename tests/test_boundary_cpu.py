"""CPU tests of the drop-in boundary: the C-ABI library loads and exports every symbol
include/b200k.h declares, argument validation answers without a GPU, descriptor bit
patterns match hand-packed golden values, and the torch op schemas equal the reference's."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200k.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200k_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from b200k import _lib
    lib = _lib.lib()
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_strerror_and_codes():
    from b200k import _lib
    assert _lib.strerror(0) == "ok"
    for code in range(-11, 0):
        assert "unknown" not in _lib.strerror(code)
    assert "unknown" in _lib.strerror(-99)


def test_argument_validation_without_gpu():
    """Validation happens before any CUDA call, so these codes come back on a CPU box too."""
    from b200k import _lib
    L = _lib.lib()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert L.b200k_gemm(p16, p16, p16, 8, 8, 8, 8, 8, 8, 7, 0, None, 0, None) == -1      # dtype
    assert L.b200k_gemm(p16, p16, p16, 0, 8, 8, 8, 8, 8, 0, 0, None, 0, None) == -2      # shape
    assert L.b200k_gemm(p16, p16, p16, 8, 8, 8, 4, 8, 8, 0, 0, None, 0, None) == -2      # lda < K
    assert L.b200k_gemm(None, p16, p16, 8, 8, 8, 8, 8, 8, 0, 0, None, 0, None) == -9     # null
    st = (ctypes.c_int64 * 3)(1024, 512, 128)
    args = lambda D, Hq=4, Hkv=2, scale=0.1, dt=0: (p16, p16, p16, p16, 1, Hq, Hkv, 4, 4, D, st, st, st, st, scale,
                                                    0, 4, dt, 0, None)
    assert L.b200k_fmha_fwd(*args(96)) == -4                                             # head_dim
    assert L.b200k_fmha_fwd(*args(128, Hq=3)) == -2                                      # Hq % Hkv
    assert L.b200k_fmha_fwd(*args(128, scale=0.0)) == -9
    assert L.b200k_fmha_fwd(*args(128, dt=5)) == -1
    bad = (ctypes.c_int64 * 3)(1024, 516, 130)
    assert L.b200k_fmha_fwd(p16, p16, p16, p16, 1, 4, 2, 4, 4, 128, bad, st, st, st, 0.1, 0, 4, 0, 0, None) == -3
    dargs = (p16, p16, p16, p16, 1, 32, 1, 1, 64, 128, st, st, st, st, 0.1, None, 0, 0, None, 0, None)
    assert L.b200k_fmha_decode_splitkv(*dargs) == -2                                     # 32 rows per KV head
    if not torch.cuda.is_available():
        assert L.b200k_device_supported() == 0
        assert L.b200k_gemm(p16, p16, p16, 8, 8, 8, 8, 8, 8, 0, 0, None, 0, None) == -10  # no GPU: loud, no fallback


def test_workspace_sizes():
    from b200k import _lib
    L = _lib.lib()
    assert L.b200k_gemm_workspace_bytes(8192, 11008, 4096, 0) == 0
    n = L.b200k_fmha_decode_workspace_bytes(64, 32, 8, 1, 32768, 128, 16)
    assert n == 64 * 8 * 4 * 16 * (128 + 2) * 4
    assert L.b200k_fmha_decode_workspace_bytes(64, 32, 8, 1, 32768, 128, 0) == \
        64 * 8 * 4 * L.b200k_fmha_decode_auto_splits(64, 8, 32768) * 130 * 4
    assert 1 <= L.b200k_fmha_decode_auto_splits(1, 1, 64) <= 64


def test_descriptor_bit_patterns():
    """Golden values packed by hand from the tcgen05 descriptor formats: shared-memory
    descriptor = start>>4 | lbo>>4 << 16 | sbo>>4 << 32 | version 1 << 46 | layout 2 << 61;
    instruction descriptor = D fp32 (1<<4) | A/B format (<<7, <<10) | A major << 15 |
    B major << 16 | N/8 << 17 | M/16 << 24."""
    from b200k import _lib
    L = _lib.lib()
    assert L.b200k_debug_smem_desc(0x400, 16, 1024) == (0x40 | (1 << 16) | (64 << 32) | (1 << 46) | (2 << 61))
    assert L.b200k_debug_smem_desc(0x12340, 8192, 1024) == (0x1234 | (512 << 16) | (64 << 32) | (1 << 46) | (2 << 61))
    # fp16, both K-major, 128x128
    assert L.b200k_debug_instr_desc(0, 0, 0, 128, 128) == ((1 << 4) | (16 << 17) | (8 << 24))
    # bf16, B MN-major, 128x256
    assert L.b200k_debug_instr_desc(1, 0, 1, 128, 256) == ((1 << 4) | (1 << 7) | (1 << 10) | (1 << 16) | (32 << 17) | (8 << 24))


def test_op_schemas_match_reference():
    """Same op names and schema strings as the reference's TORCH_LIBRARY blocks
    (kernels/gemm/pkg/gemm_unified/csrc/gemm_kernel.cu:9-27,
     kernels/fmha/pkg/fmha_unified/csrc/fmha_kernel.cu:9-18)."""
    import fmha_unified
    import gemm_unified
    for i in range(17):
        op = getattr(torch.ops.gemm_unified, f"finegemm_{i}").default
        assert str(op._schema) == f"gemm_unified::finegemm_{i}(Tensor a, Tensor b) -> Tensor"
    for i in range(8):
        op = getattr(torch.ops.fmha_unified, f"finefmha_{i}").default
        assert str(op._schema) == (f"fmha_unified::finefmha_{i}(Tensor q, Tensor k, Tensor v, bool causal, "
                                   "bool is_decode, int decode_length) -> Tensor")
    assert hasattr(gemm_unified, "_C") and hasattr(gemm_unified, "ops")
    assert hasattr(fmha_unified, "_C") and hasattr(fmha_unified, "ops")
    assert gemm_unified.ops.__all__ == ["fine_gemm"]


def test_no_cpu_fallback():
    """CPU tensors are refused: there is no eager or oracle path behind the ops."""
    import fmha_unified
    import gemm_unified
    a = torch.zeros(8, 8, dtype=torch.float16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        gemm_unified.ops.fine_gemm(a, a, 0)
    q = torch.zeros(1, 1, 8, 128, dtype=torch.float16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        fmha_unified.ops.fine_fmha(q, q, q, True, False, 0)
    from b200k import gemm
    with pytest.raises(RuntimeError):
        gemm.gemm(a, a)


def test_product_never_imports_oracle():
    pkg = os.path.join(ROOT, "understanding-gpu-architecture-implications-on-llm-serving-workloads_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, os.path.join(dirpath, f)
