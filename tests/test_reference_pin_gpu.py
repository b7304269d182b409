"""Pins the oracle to the reference itself: the reference's own CUDA rungs, compiled for sm_100 from
the reference checkout by oracle/build_ref_ladder.py (oracle/_ref/*.so), are run on the inputs of the
reference's correctness scripts and their outputs are compared with the oracle inside the
tolerances those scripts accept:

  GEMM  kernels/gemm/test/correct.py:5-16   seed 0, a, b = randn(256, 256) fp16, rtol = atol = 1e-1
  FMHA  kernels/fmha/test/correct.py:26-55  seed 42, randn * 0.1, B=1, 1/1 and 4/1 heads, s=128,
                                            d=128, fp16, atol 5e-2 (causal and full)

and the library is compared with the oracle on the very same tensors inside the build's own,
tighter bars (relative Frobenius 1e-2, max-abs 2e-3).  The reference rungs run in a child process
(oracle/run_ref_check.py): their library registers the op namespaces this repo's packages
register.  Skipped when oracle/_ref/ was not built."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")

FMHA_CASES = {"mha_causal": (False, True), "mha_full": (False, False),
              "gqa_causal": (True, True), "gqa_full": (True, False)}


def _reference_check_inputs():
    torch.manual_seed(0)   # kernels/gemm/test/correct.py:5-8
    arrays = {"gemm_a": torch.randn(256, 256, dtype=torch.half).numpy(),
              "gemm_b": torch.randn(256, 256, dtype=torch.half).numpy()}
    for name, (gqa, causal) in FMHA_CASES.items():
        torch.manual_seed(42)  # kernels/fmha/test/correct.py:39-47 (drawn per call of correct())
        n_head = 4 if gqa else 1
        kv_head = n_head // 4 if gqa else n_head
        for x, heads in (("q", n_head), ("k", kv_head), ("v", kv_head)):
            arrays[f"{name}.{x}"] = (torch.randn(1, heads, 128, 128, dtype=torch.half) * 0.1).numpy()
        arrays[f"{name}.causal"] = np.array(causal)
    return arrays


@pytest.fixture(scope="module")
def reference_outputs(tmp_path_factory):
    if not (os.path.exists(os.path.join(REF_DIR, "ref_gemm_unified.so"))
            or os.path.exists(os.path.join(REF_DIR, "ref_fmha_unified.so"))):
        pytest.skip("oracle/_ref/ not built (python oracle/build_ref_ladder.py <reference checkout>)")
    d = tmp_path_factory.mktemp("refpin")
    inp, outp = str(d / "in.npz"), str(d / "out.npz")
    arrays = _reference_check_inputs()
    np.savez(inp, **arrays)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_ref_check.py"), inp, outp],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    return arrays, np.load(outp)


def test_golden_fixtures_hold_the_reference_inputs(reference_outputs):
    """The committed fixtures (tests/golden/) were drawn by the same recipe: same bits."""
    arrays, _ = reference_outputs
    gold = os.path.join(ROOT, "tests", "golden")
    z = np.load(os.path.join(gold, "gemm_seed0_256.npz"))
    assert np.array_equal(z["a"], arrays["gemm_a"]) and np.array_equal(z["b"], arrays["gemm_b"])
    z = np.load(os.path.join(gold, "fmha_seed42_gqa_causal_f16.npz"))
    assert all(np.array_equal(z[x], arrays[f"gqa_causal.{x}"]) for x in "qkv")


def test_gemm_oracle_vs_reference_rungs_vs_library(reference_outputs, cuda_device):
    arrays, ref = reference_outputs
    if not bool(ref["have_gemm"]):
        pytest.skip("ref_gemm_unified.so not built")
    import gemm_unified
    a, b = torch.from_numpy(arrays["gemm_a"]), torch.from_numpy(arrays["gemm_b"])
    want = oracle.gemm_ref(a, b)
    for rung in (8, 9, 10, 11):
        got = torch.from_numpy(ref[f"gemm_{rung}"]).float()
        # the reference's own acceptance window, with the oracle in the place of `a @ b`
        assert torch.allclose(got, want, rtol=1e-1, atol=1e-1), rung
        # what the rungs actually achieve with fp16 accumulation over K = 256 (observed on B200: 6.0e-4,
        # max-abs 0.087; the library on the same tensors: 2.1e-4)
        assert oracle.rel_frobenius(got, want) <= 2e-3, (rung, oracle.rel_frobenius(got, want))
    for idx in (0, 8, 11, 12):
        c = gemm_unified.ops.fine_gemm(a.to(cuda_device), b.to(cuda_device), idx)
        assert oracle.rel_frobenius(c, want) <= oracle.GEMM_REL_FRO_TOL
        assert torch.allclose(c.cpu().float(), want, rtol=1e-1, atol=1e-1)
        # library and reference rung agree inside the reference's window as well
        assert torch.allclose(c.cpu().float(), torch.from_numpy(ref["gemm_11"]).float(), rtol=1e-1, atol=1e-1)


@pytest.mark.parametrize("case", sorted(FMHA_CASES))
def test_fmha_oracle_vs_reference_rungs_vs_library(reference_outputs, cuda_device, case):
    arrays, ref = reference_outputs
    if not bool(ref["have_fmha"]):
        pytest.skip("ref_fmha_unified.so not built")
    import fmha_unified
    q, k, v = (torch.from_numpy(arrays[f"{case}.{x}"]) for x in "qkv")
    causal = FMHA_CASES[case][1]
    want = oracle.fmha_ref(q, k, v, causal=causal)
    for rung in (2, 3, 4):
        got = torch.from_numpy(ref[f"{case}.fmha_{rung}"]).float()
        assert not torch.isnan(got).any()
        # kernels/fmha/test/correct.py:55: allclose(rtol=0, atol=5e-2)
        assert torch.allclose(got, want, rtol=0, atol=5e-2), (rung, oracle.max_abs(got, want))
        # what the rungs actually achieve on these inputs (observed on B200: 1.7e-4 .. 2.9e-4 with their
        # fp16 softmax state; the library: 1.1e-5 .. 7.2e-5)
        assert oracle.max_abs(got, want) <= 1e-3, (rung, oracle.max_abs(got, want))
    # the library on the same tensors, inside its own bar, through the reference-facing wrapper
    for idx in (2, 4, 5):
        o = fmha_unified.ops.fine_fmha(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal, False, idx)
        assert oracle.max_abs(o, want) <= oracle.FMHA_MAX_ABS_TOL
        assert torch.allclose(o.cpu().float(), torch.from_numpy(ref[f"{case}.fmha_4"]).float(), rtol=0, atol=5e-2)
