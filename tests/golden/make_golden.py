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

`torch_attn` is not restated here: it is IMPORTED from the reference checkout
(kernels/fmha/test/perf.py:10-24, the same function as kernels/fmha/test/correct.py:10-24;
perf.py keeps its sweep behind `if __name__ == "__main__"`, correct.py runs a GPU check
at import, so perf.py is the importable one).  Its module-level `import fmha_unified`
resolves to the drop-in package of this repo; nothing of that package is called.

Run from the repo root:  python tests/golden/make_golden.py /path/to/reference
(or with REFERENCE_ROOT set).  The fixtures travel with the repo; the reference
checkout is only needed to regenerate them.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(OUT))
PKG = os.path.join(ROOT, "understanding-gpu-architecture-implications-on-llm-serving-workloads_b200")


def load_reference_torch_attn(reference_root: str):
    """The reference test scripts' oracle function, imported from the checkout."""
    path = os.path.join(reference_root, "kernels", "fmha", "test", "perf.py")
    if not os.path.exists(path):
        sys.exit(f"{path} not found: pass the reference checkout as the first argument or set REFERENCE_ROOT")
    if PKG not in sys.path:
        sys.path.insert(0, PKG)  # perf.py imports fmha_unified at module level
    spec = importlib.util.spec_from_file_location("reference_fmha_perf", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.torch_attn


torch_attn = None  # bound in __main__


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
    torch_attn = load_reference_torch_attn(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", ""))
    gemm_case()
    fmha_case("fmha_seed42_mha_causal_f16", False, True, False, torch.half)
    fmha_case("fmha_seed42_gqa_causal_f16", True, True, False, torch.half)
    fmha_case("fmha_seed42_gqa_full_bf16", True, False, False, torch.bfloat16)
    fmha_case("fmha_seed42_gqa_decode_f16", True, False, True, torch.half)
    print(sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))
