"""The two bindings of the reference's torch ops - the compiled TORCH_LIBRARY shim (C++ over the C ABI,
the reference's own form: kernels/gemm/pkg/gemm_unified/csrc/gemm_kernel.cu:9-27) and the Python/ctypes
registration - run the same calls in a process each (one process holds one binding) and must return the
same bits, raise the same kinds of error, and meet the oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _child(binding, path):
    env = dict(os.environ, B200K_BINDING=binding)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "binding_child.py"), path], env=env,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    return np.load(path)


def test_compiled_and_ctypes_bindings_agree(cuda_device, tmp_path):
    from b200k import _binding, inputs
    if not _binding.SHIM_PATH.exists():
        pytest.fail(f"{_binding.SHIM_PATH} was not built")
    compiled = _child("compiled", str(tmp_path / "compiled.npz"))
    ctypes_ = _child("ctypes", str(tmp_path / "ctypes.npz"))
    assert str(compiled["binding"]) == "compiled" and str(ctypes_["binding"]) == "ctypes"
    keys = sorted(k for k in compiled.files if k not in ("binding", "errors"))
    assert keys == sorted(k for k in ctypes_.files if k not in ("binding", "errors"))
    for key in keys:
        assert np.array_equal(compiled[key], ctypes_[key]), key
    assert list(compiled["errors"]) == list(ctypes_["errors"])
    assert all(not e.endswith(":none") for e in compiled["errors"]), list(compiled["errors"])
    # and the compiled binding's results meet the oracle
    a, b = inputs.gemm_llm(300, 520, 264, torch.bfloat16, seed=3)
    ref = oracle.gemm_ref(a, b)
    for idx in (0, 8, 9, 10, 11, 12):
        got = torch.from_numpy(compiled[f"gemm_{idx}"]).view(torch.bfloat16)
        assert oracle.rel_frobenius(got, ref) <= oracle.GEMM_REL_FRO_TOL
    q, k, v = inputs.fmha_inputs(2, 8, 2, 300, 300, 128, torch.float16, seed=5)
    want = oracle.fmha_ref(q, k, v, causal=True)
    for key in ("prefill_causal", "prefill_bshd"):
        got = torch.from_numpy(compiled[key]).view(torch.float16)
        assert oracle.max_abs(got, want) <= oracle.FMHA_MAX_ABS_TOL
    q, k, v = inputs.fmha_inputs(2, 32, 1, 1, 700, 64, torch.float16, seed=7)
    got = torch.from_numpy(compiled["decode_mqa"]).view(torch.float16)
    assert oracle.max_abs(got, oracle.fmha_ref(q, k, v)) <= oracle.FMHA_MAX_ABS_TOL
    q, k, v = inputs.fmha_inputs(3, 32, 8, 1, 1000, 128, torch.bfloat16, seed=6)
    ok, err = oracle.fmha_within_tolerance(torch.from_numpy(compiled["varlen"]).view(torch.bfloat16),
                                           oracle.fmha_ref(q, k, v, kv_lens=[1000, 1, 513]))
    assert ok, err
