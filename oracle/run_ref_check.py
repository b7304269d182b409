"""Runs the reference's own kernel rungs (built for sm_100 by oracle/build_ref_ladder.py into
oracle/_ref/) on the inputs of the reference's correctness scripts and saves what they return.
TEST INFRASTRUCTURE ONLY: tests/test_reference_pin_gpu.py starts this file in a process of its own
(the reference libraries register the op namespaces gemm_unified / fmha_unified, which the drop-in
packages register too, so the two cannot share a process) and compares the saved outputs with the
oracle.

    python oracle/run_ref_check.py inputs.npz outputs.npz

inputs.npz holds fp16 arrays `gemm_a`, `gemm_b` (kernels/gemm/test/correct.py:5-8: seed 0, 256 x 256)
and, per attention case c, `c.q`, `c.k`, `c.v`, `c.causal` (kernels/fmha/test/correct.py:26-47:
seed 42, randn * 0.1, B=1, 1/1 or 4/1 heads, s=128, d=128).  Only these shapes are run: multiples of
128 in every dimension, which is what the tensor-core rungs (no bounds checks) are written for.
The ops are called exactly as the reference's Python wrappers call them
(kernels/gemm/pkg/gemm_unified/ops.py:11-13, kernels/fmha/pkg/fmha_unified/ops.py:27 with
decode_length = k.size(2)).  A missing library is reported in the output file, not an error.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GEMM_RUNGS = (8, 9, 10, 11)
FMHA_RUNGS = (2, 3, 4)


def main(inp: str, outp: str) -> int:
    z = np.load(inp)
    out = {}
    dev = torch.device("cuda", 0)
    gemm_so = os.path.join(HERE, "_ref", "ref_gemm_unified.so")
    fmha_so = os.path.join(HERE, "_ref", "ref_fmha_unified.so")
    out["have_gemm"] = np.array(os.path.exists(gemm_so))
    out["have_fmha"] = np.array(os.path.exists(fmha_so))
    if out["have_gemm"]:
        torch.ops.load_library(gemm_so)
        a = torch.from_numpy(z["gemm_a"]).to(dev)
        b = torch.from_numpy(z["gemm_b"]).to(dev)
        for rung in GEMM_RUNGS:
            c = getattr(torch.ops.gemm_unified, f"finegemm_{rung}").default(a, b)
            torch.cuda.synchronize()
            out[f"gemm_{rung}"] = c.cpu().numpy()
    if out["have_fmha"]:
        torch.ops.load_library(fmha_so)
        cases = sorted({key.split(".")[0] for key in z.files if "." in key})
        for case in cases:
            q, k, v = (torch.from_numpy(z[f"{case}.{x}"]).to(dev) for x in ("q", "k", "v"))
            causal = bool(z[f"{case}.causal"])
            for rung in FMHA_RUNGS:
                o = getattr(torch.ops.fmha_unified, f"finefmha_{rung}").default(q, k, v, causal, False, k.size(2))
                torch.cuda.synchronize()
                out[f"{case}.fmha_{rung}"] = o.cpu().numpy()
    np.savez(outp, **out)
    return 0


if __name__ == "__main__":
    if len(sys.argv) != 3:
        sys.exit("usage: run_ref_check.py inputs.npz outputs.npz")
    sys.exit(main(sys.argv[1], sys.argv[2]))
