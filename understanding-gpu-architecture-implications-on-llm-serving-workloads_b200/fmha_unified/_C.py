"""Registers the reference's FMHA op schema and routes it to libb200k.so.

Same op names and signatures as the reference's TORCH_LIBRARY block
(kernels/fmha/pkg/fmha_unified/csrc/fmha_kernel.cu:9-18):
`fmha_unified::finefmha_{0..7}(Tensor q, Tensor k, Tensor v, bool causal,
bool is_decode, int decode_length) -> Tensor`.  Indices 0..5 (every index the
reference implements for NVIDIA) get a CUDA implementation; 6 and 7 stay
declared only, as in the reference.

Argument meaning follows the reference launchers
(kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_4_nv.cu:395-443): q [B,Hq,Nq,d],
k, v [B,Hkv,Nkv,d]; `is_decode` requires `causal == False` (:415-417) and masks
keys beyond `decode_length`; with `is_decode == False` `decode_length` only
describes padding the reference's Python wrapper added and is applied as the
valid key count as well.  Every index accepts fp16 and bf16 and d in {64, 128}.
One op is added, `finefmha_decode_varlen(q, k, v, kv_lens)`, because a scalar
`decode_length` cannot carry per-sequence KV lengths.

The registration itself lives in C++ when the compiled binding has been built
(torch_shim/ops_shim.cpp, loaded here), otherwise in this module over ctypes; see b200k/_binding.py.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from b200k import _binding, fmha as _fmha  # noqa: E402

NUM_DECLARED = 8
NUM_IMPLEMENTED = 6
# decode-shaped calls (few query rows) go to the split-KV kernels
DECODE_MAX_SQ = 8

BINDING = _binding.binding()  # "compiled": the C++ TORCH_LIBRARY blocks are loaded and nothing is defined here


def _finefmha(q, k, v, causal: bool, is_decode: bool, decode_length: int):
    if is_decode and causal:
        # kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_4_nv.cu:415-417
        raise RuntimeError("is_decode and causal cannot be true at the same time")
    n_kv = k.size(2)
    kv_len = n_kv if decode_length <= 0 else min(int(decode_length), n_kv)
    if is_decode and q.size(2) <= DECODE_MAX_SQ:
        lens = None
        if kv_len != n_kv:
            lens = torch.full((q.size(0),), kv_len, dtype=torch.int32, device=q.device)
        return _fmha.fmha_decode(q, k, v, kv_lens=lens)
    return _fmha.fmha_fwd(q, k, v, causal=causal, kv_len=kv_len)


def _finefmha_decode_varlen(q, k, v, kv_lens):
    return _fmha.fmha_decode(q, k, v, kv_lens=kv_lens)


if BINDING == "ctypes":
    _library = torch.library.Library("fmha_unified", "DEF")
    for _i in range(NUM_DECLARED):
        _library.define(f"finefmha_{_i}(Tensor q, Tensor k, Tensor v, bool causal, bool is_decode, "
                        "int decode_length) -> Tensor")
    _library.define("finefmha_decode_varlen(Tensor q, Tensor k, Tensor v, Tensor kv_lens) -> Tensor")
    for _i in range(NUM_IMPLEMENTED):
        _library.impl(f"finefmha_{_i}", _finefmha, "CUDA")
    _library.impl("finefmha_decode_varlen", _finefmha_decode_varlen, "CUDA")
