"""Child process of tests/test_binding_gpu.py: runs the reference-facing ops through the binding
named by B200K_BINDING on seeded inputs and saves the raw 16-bit results."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "understanding-gpu-architecture-implications-on-llm-serving-workloads_b200"))

import fmha_unified  # noqa: E402
import gemm_unified  # noqa: E402
from b200k import inputs  # noqa: E402


def main(out_path: str) -> int:
    dev = torch.device("cuda", 0)
    res = {"binding": np.array(gemm_unified._C.BINDING)}
    a, b = inputs.gemm_llm(300, 520, 264, torch.bfloat16, seed=3)
    for idx in (0, 8, 9, 10, 11, 12):
        res[f"gemm_{idx}"] = gemm_unified.ops.fine_gemm(a.to(dev), b.to(dev), idx).view(torch.int16).cpu().numpy()
    a, b = inputs.gemm_llm(16, 1024, 512, torch.float16, seed=4)
    res["gemm_skinny"] = gemm_unified.ops.fine_gemm(a.to(dev), b.to(dev), 12).view(torch.int16).cpu().numpy()
    q, k, v = inputs.fmha_inputs(2, 8, 2, 300, 300, 128, torch.float16, seed=5)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    res["prefill_causal"] = fmha_unified.ops.fine_fmha(qd, kd, vd, True, False, 5).view(torch.int16).cpu().numpy()
    res["prefill_full"] = fmha_unified.ops.fine_fmha(qd, kd, vd, False, False, 2).view(torch.int16).cpu().numpy()
    # bshd storage viewed as bhsd
    qs, ks, vs = inputs.fmha_inputs(2, 8, 2, 300, 300, 128, torch.float16, device=dev, seed=5, layout="bshd")
    res["prefill_bshd"] = fmha_unified.ops.fine_fmha(qs, ks, vs, True, False, 5).view(torch.int16).cpu().numpy()
    q, k, v = inputs.fmha_inputs(3, 32, 8, 1, 1000, 128, torch.bfloat16, seed=6)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    res["decode"] = fmha_unified.ops.fine_fmha(qd, kd, vd, False, True, 4).view(torch.int16).cpu().numpy()
    lens = torch.tensor([1000, 1, 513], dtype=torch.int32, device=dev)
    res["varlen"] = fmha_unified.ops.fine_fmha_decode_varlen(qd, kd, vd, lens).view(torch.int16).cpu().numpy()
    q, k, v = inputs.fmha_inputs(2, 32, 1, 1, 700, 64, torch.float16, seed=7)  # MQA: 32 rows per KV head
    res["decode_mqa"] = fmha_unified.ops.fine_fmha(q.to(dev), k.to(dev), v.to(dev), False, True,
                                                   0).view(torch.int16).cpu().numpy()
    errors = []
    for name, call in (
            ("causal_and_decode", lambda: fmha_unified.ops.fine_fmha(qd, kd, vd, True, True, 0)),
            ("declared_only_fmha", lambda: fmha_unified.ops.fine_fmha(qd, kd, vd, True, False, 6)),
            ("declared_only_gemm", lambda: gemm_unified.ops.fine_gemm(a.to(dev), b.to(dev), 13)),
            ("fp32", lambda: gemm_unified.ops.fine_gemm(a.to(dev).float(), b.to(dev).float(), 0)),
            ("shape", lambda: gemm_unified.ops.fine_gemm(a.to(dev), a.to(dev), 0)),
            ("head_dim", lambda: fmha_unified.ops.fine_fmha(qd[..., :32], kd[..., :32], vd[..., :32], True, False, 0))):
        try:
            call()
            errors.append(f"{name}:none")
        except (RuntimeError, NotImplementedError) as exc:
            errors.append(f"{name}:{type(exc).__name__}")
    res["errors"] = np.array(errors)
    torch.cuda.synchronize()
    np.savez(out_path, **res)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
