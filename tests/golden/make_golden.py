"""Generates tests/golden/*.npz: outputs of the reference test scripts' own oracle
functions on the reference's seeds and shapes, computed on CPU in this build's
container.  The reference ships no golden vectors; its checks call torch at run
time, and these fixtures freeze what those calls return so the repo's oracle
(oracle/oracle.py, oracle/oracle_c.c) can be pinned without the reference tree.

  GEMM  (kernels/gemm/test/correct.py:5-16): torch.manual_seed(0); a, b =
        randn(256, 256) fp16; expected = a @ b.
  FMHA  (kernels/fmha/test/correct.py:10-24,26-47): torch.manual_seed(42); B=1,
        heads 1/1 or 4/1 (GQA), s=128 (q_len 1 for decode), d=128, inputs
        randn * 0.1; expected = `torch_attn`, i.e. repeat_kv followed by
        F.scaled_dot_product_attention(q, k, v, is_causal=...).  (The script's
        active line compares against raw QK^T instead, a debugging leftover at :52;
        the function it defines and names as the oracle is what is frozen here.)

Run from the repo root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch
from torch.nn import functional as F

OUT = os.path.dirname(os.path.abspath(__file__))


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    # what kernels/fmha/test/correct.py:11-20 does: each KV head repeated n_rep times in place
    return x if n_rep == 1 else torch.repeat_interleave(x, n_rep, dim=1)


def torch_attn(q, k, v, is_causal):
    if q.size(1) != k.size(1):
        k, v = repeat_kv(k, 4), repeat_kv(v, 4)
    return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal)


def gemm_case():
    torch.manual_seed(0)
    a = torch.randn(256, 256, dtype=torch.half)
    b = torch.randn(256, 256, dtype=torch.half)
    expected = a.float() @ b.float()
    np.savez_compressed(os.path.join(OUT, "gemm_seed0_256.npz"), a=a.numpy(), b=b.numpy(),
                        expected=expected.numpy())


def fmha_case(name, gqa, causal, decode, dtype):
    torch.manual_seed(42)
    n_head = 4 if gqa else 1
    kv_head = n_head // 4 if gqa else n_head
    s, d = 128, 128
    q_len = 1 if decode else s
    q = torch.randn(1, n_head, q_len, d, dtype=dtype) * 0.1
    k = torch.randn(1, kv_head, s, d, dtype=dtype) * 0.1
    v = torch.randn(1, kv_head, s, d, dtype=dtype) * 0.1
    expected = torch_attn(q.float(), k.float(), v.float(), causal)
    as_np = (lambda t: t.view(torch.int16).numpy()) if dtype == torch.bfloat16 else (lambda t: t.numpy())
    np.savez_compressed(os.path.join(OUT, name + ".npz"), q=as_np(q), k=as_np(k), v=as_np(v),
                        expected=expected.numpy(), causal=np.array(causal), bf16=np.array(dtype == torch.bfloat16))


if __name__ == "__main__":
    gemm_case()
    fmha_case("fmha_seed42_mha_causal_f16", False, True, False, torch.half)
    fmha_case("fmha_seed42_gqa_causal_f16", True, True, False, torch.half)
    fmha_case("fmha_seed42_gqa_full_bf16", True, False, False, torch.bfloat16)
    fmha_case("fmha_seed42_gqa_decode_f16", True, False, True, torch.half)
    print(sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))
