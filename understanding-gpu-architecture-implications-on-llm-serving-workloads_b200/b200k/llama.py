"""Llama-shaped decoder stack on the B200 kernels, with randomly initialised weights, and a
generation-style timing harness.

    python -m b200k.llama [--layers 32] [--batch 8] [--prompt-len 2048] [--gen-len 32] [--baseline]

The reference times HuggingFace `generate()` on downloaded checkpoints
(benchmarks/huggingface-cuda/hf-gen.py:46-130: prefill latency from forward hooks,
benchmarks/utils.py:75-98; prefill / decode / total tokens per second) and routes attention to
`fmha_unified.ops.fine_fmha` in a forked modeling file
(benchmarks/flashattn-cuda/modeling_llama.py:654-704), while its linear layers stay on cuBLAS.
No checkpoint, tokenizer or dataset is available or reproduced here: the model below has the
Llama-2-7B *shape* with N(0, 0.02) weights and is fed random token ids, which is enough to
time the same prefill / decode phases with every projection and the attention on this
library:
    q/k/v   one GEMM over the fused QKV weight
    RoPE    torch element-wise (not part of the reference's kernel packages)
    prefill fmha_fwd, causal, reading q as stored [B,S,H,D] and K/V from the cache (no copies)
    decode  fmha_decode (split-KV) over the padded cache with per-sequence lengths
    o_proj, down_proj   GEMM with the residual add fused into the epilogue
    gate/up one GEMM over the column-interleaved weight with SiLU(gate)*up fused
`--baseline` times the same stack with torch.matmul and scaled_dot_product_attention.

Decode steps are launch-bound from Python (about ten small kernels per layer), so by default the
step is captured once in a CUDA graph and replayed (`--no-graph` keeps the eager loop): position,
per-sequence lengths and the token fed back all live in device tensors that the captured step
updates in place, the cache write is an index_copy_ at the device-side position, and the decode
attention runs on the library's allocation-free entry point, so a replay touches no host state.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import fmha, gemm


@dataclass
class LlamaConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    intermediate: int = 11008
    n_layers: int = 32
    vocab: int = 32000
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0


def _rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,D]; cos/sin [B,S,1,D/2] (rotate-half convention)."""
    d = x.size(-1) // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


class SyntheticLlama:
    """Weights N(0, 0.02) of a Llama-shaped model; `use_library=False` swaps every kernel of this
    library for its torch counterpart (the comparator, also used by the numerics test)."""

    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device="cuda", seed: int = 0, use_library: bool = True):
        self.cfg, self.dtype, self.device, self.lib = cfg, dtype, torch.device(device), use_library
        g = torch.Generator(device=self.device).manual_seed(seed)

        def w(*shape):
            t = torch.empty(shape, dtype=dtype, device=self.device)
            t.normal_(0.0, 0.02, generator=g)
            return t

        H, D, F_ = cfg.hidden, cfg.head_dim, cfg.intermediate
        self.qkv_cols = (cfg.n_heads + 2 * cfg.n_kv_heads) * D
        self.embed = w(cfg.vocab, H)
        self.layers = []
        for _ in range(cfg.n_layers):
            gate, up = w(H, F_), w(H, F_)
            self.layers.append({
                "wqkv": w(H, self.qkv_cols), "wo": w(cfg.n_heads * D, H),
                "w_gate": gate, "w_up": up, "w_gate_up": gemm.interleave_gate_up(gate, up) if use_library else None,
                "w_down": w(F_, H),
                "norm1": torch.ones(H, dtype=dtype, device=self.device),
                "norm2": torch.ones(H, dtype=dtype, device=self.device)})
            if use_library:
                self.layers[-1]["w_gate"] = self.layers[-1]["w_up"] = None  # only the interleaved copy is kept
        self.norm_f = torch.ones(H, dtype=dtype, device=self.device)
        self.lm_head = w(H, cfg.vocab)
        self.k_cache = self.v_cache = None

    # -------------------------------------------------------------------- cache
    def alloc_cache(self, batch: int, max_len: int) -> None:
        c = self.cfg
        shape = (c.n_layers, batch, c.n_kv_heads, max_len, c.head_dim)
        self.k_cache = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.v_cache = torch.zeros(shape, dtype=self.dtype, device=self.device)

    def _angles(self, positions: torch.Tensor):
        c = self.cfg
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=self.device, dtype=torch.float32) / c.head_dim))
        ang = positions.float()[..., None] * inv  # [B,S,D/2]
        return ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]

    # -------------------------------------------------------------------- kernels or comparators
    def _mm(self, a, w):
        return gemm.gemm(a, w) if self.lib else torch.matmul(a, w)

    def _mm_add(self, a, w, r):
        return gemm.gemm_add(a, w, r) if self.lib else torch.matmul(a, w) + r

    def _mlp_in(self, h, layer):
        if self.lib:
            return gemm.gemm_swiglu(h, layer["w_gate_up"])
        return F.silu(torch.matmul(h, layer["w_gate"])) * torch.matmul(h, layer["w_up"])

    # -------------------------------------------------------------------- forward
    def forward(self, tokens: torch.Tensor, start: int, kv_lens: torch.Tensor | None = None) -> torch.Tensor:
        """tokens [B,S] at positions start..start+S-1 (prefill: start = 0, S = prompt; decode: S = 1).
        Returns logits of the last position [B, vocab]."""
        c = self.cfg
        B, S = tokens.shape
        D, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        x = self.embed[tokens.reshape(-1)]  # [B*S, hidden]
        pos = torch.arange(start, start + S, device=self.device)[None, :].expand(B, S)
        cos, sin = self._angles(pos)
        end = start + S
        for li, layer in enumerate(self.layers):
            h = _rms_norm(x, layer["norm1"], c.rms_eps)
            qkv = self._mm(h, layer["wqkv"]).view(B, S, Hq + 2 * Hkv, D)
            q = _rope(qkv[:, :, :Hq], cos, sin)                       # [B,S,Hq,D]
            k = _rope(qkv[:, :, Hq:Hq + Hkv], cos, sin)
            v = qkv[:, :, Hq + Hkv:]
            kc, vc = self.k_cache[li], self.v_cache[li]               # [B,Hkv,Smax,D]
            kc[:, :, start:end] = k.transpose(1, 2)
            vc[:, :, start:end] = v.transpose(1, 2)
            qv = q.transpose(1, 2)                                    # [B,Hq,S,D] view of [B,S,Hq,D] storage
            attn = torch.empty((B, S, Hq, D), dtype=self.dtype, device=self.device)
            av = attn.transpose(1, 2)
            if self.lib:
                if S == 1:
                    lens = kv_lens if kv_lens is not None else torch.full((B,), end, dtype=torch.int32, device=self.device)
                    fmha.fmha_decode(qv, kc, vc, kv_lens=lens, out=av)
                else:
                    fmha.fmha_fwd(qv, kc, vc, causal=True, kv_len=end, out=av)
            else:
                av.copy_(F.scaled_dot_product_attention(qv, kc[:, :, :end], vc[:, :, :end], is_causal=S > 1,
                                                        enable_gqa=Hq != Hkv))
            x = self._mm_add(attn.view(B * S, Hq * D), layer["wo"], x)
            h = _rms_norm(x, layer["norm2"], c.rms_eps)
            x = self._mm_add(self._mlp_in(h, layer), layer["w_down"], x)
        x = _rms_norm(x.view(B, S, -1)[:, -1], self.norm_f, c.rms_eps)
        return self._mm(x.contiguous(), self.lm_head)

    def _decode_step(self, st: dict) -> None:
        """One greedy decode step with all step state on the device (capturable in a CUDA graph):
        st["tok"] [B,1] is consumed and overwritten with the next token, st["pos"] (int64 [1]) and
        st["lens"] (int32 [B]) advance by one, the new token is also written to st["out"][:, pos+1]."""
        c = self.cfg
        tok, pos, lens = st["tok"], st["pos"], st["lens"]
        B = tok.size(0)
        D, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        x = self.embed.index_select(0, tok.reshape(-1))
        cos, sin = self._angles(pos.view(1, 1).expand(B, 1))
        lens.add_(1)  # the key written below counts
        for li, layer in enumerate(self.layers):
            h = _rms_norm(x, layer["norm1"], c.rms_eps)
            qkv = self._mm(h, layer["wqkv"]).view(B, 1, Hq + 2 * Hkv, D)
            q = _rope(qkv[:, :, :Hq], cos, sin)
            k = _rope(qkv[:, :, Hq:Hq + Hkv], cos, sin)
            v = qkv[:, :, Hq + Hkv:]
            kc, vc = self.k_cache[li], self.v_cache[li]
            kc.index_copy_(2, pos, k.transpose(1, 2))
            vc.index_copy_(2, pos, v.transpose(1, 2))
            attn = torch.empty((B, 1, Hq, D), dtype=self.dtype, device=self.device)
            av = attn.transpose(1, 2)
            if self.lib:
                fmha.fmha_decode(q.transpose(1, 2), kc, vc, kv_lens=lens, out=av, static_scratch=st["static_scratch"])
            else:
                # comparator: lengths are uniform here, so the valid prefix is a mask over the padded cache
                mask = (torch.arange(kc.size(2), device=self.device)[None, :] < lens[:, None].long())[:, None, None, :]
                av.copy_(F.scaled_dot_product_attention(q.transpose(1, 2), kc, vc, attn_mask=mask, enable_gqa=Hq != Hkv))
            x = self._mm_add(attn.view(B, Hq * D), layer["wo"], x)
            h = _rms_norm(x, layer["norm2"], c.rms_eps)
            x = self._mm_add(self._mlp_in(h, layer), layer["w_down"], x)
        x = _rms_norm(x, self.norm_f, c.rms_eps)
        nxt = self._mm(x.contiguous(), self.lm_head).argmax(-1, keepdim=True)
        pos.add_(1)
        st["out"].index_copy_(1, pos, nxt)
        tok.copy_(nxt)

    @torch.no_grad()
    def generate_graphed(self, prompt: torch.Tensor, gen_len: int):
        """Greedy decoding with the decode step captured in a CUDA graph; same return values as
        `generate`.  The capture (and its warm-up step on a side stream) happens before the timed
        region and leaves the step state untouched: it runs on scratch copies of the state."""
        B, S = prompt.shape
        self.alloc_cache(B, S + gen_len)
        dev = self.device
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        out = torch.zeros((B, S + gen_len), dtype=torch.long, device=dev)
        out[:, :S] = prompt
        st = {"tok": torch.zeros((B, 1), dtype=torch.long, device=dev), "pos": torch.zeros(1, dtype=torch.long, device=dev),
              "lens": torch.zeros(B, dtype=torch.int32, device=dev), "out": out,
              "static_scratch": bool(self.lib)}  # the allocation-free entry point takes any size with its own split choice

        def reset(first_tok):
            st["tok"].copy_(first_tok)
            st["pos"].fill_(S)      # position of the token in st["tok"]
            st["lens"].fill_(S)     # keys in the cache before that token is appended
        graph = None
        if gen_len > 1:
            # capture on dummy state (token 0 at position S): the cache slot it writes is rewritten by the real step
            reset(torch.zeros((B, 1), dtype=torch.long, device=dev))
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._decode_step(st)
            torch.cuda.current_stream().wait_stream(side)
            reset(torch.zeros((B, 1), dtype=torch.long, device=dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._decode_step(st)
            torch.cuda.synchronize()
        e[0].record()
        nxt = self.forward(prompt, 0).argmax(-1, keepdim=True)
        e[1].record()
        out[:, S:S + 1] = nxt
        reset(nxt)
        for _ in range(1, gen_len):
            graph.replay()
        e[2].record()
        torch.cuda.synchronize()
        return out, e[0].elapsed_time(e[1]) / 1e3, e[1].elapsed_time(e[2]) / 1e3

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, gen_len: int):
        """Greedy decoding; returns (tokens [B, prompt+gen], prefill seconds, decode seconds) timed with
        CUDA events (the reference's hooks use host clocks around synchronisations)."""
        B, S = prompt.shape
        self.alloc_cache(B, S + gen_len)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        out = [prompt]
        e[0].record()
        nxt = self.forward(prompt, 0).argmax(-1, keepdim=True)
        e[1].record()
        out.append(nxt)
        for t in range(1, gen_len):
            nxt = self.forward(nxt, S + t - 1).argmax(-1, keepdim=True)
            out.append(nxt)
        e[2].record()
        torch.cuda.synchronize()
        return torch.cat(out, dim=1), e[0].elapsed_time(e[1]) / 1e3, e[1].elapsed_time(e[2]) / 1e3


def run(cfg: LlamaConfig, batch: int, prompt_len: int, gen_len: int, use_library: bool, dtype=torch.bfloat16,
        graph: bool = True) -> dict:
    model = SyntheticLlama(cfg, dtype=dtype, use_library=use_library)
    g = torch.Generator(device=model.device).manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=g, device=model.device)
    gen = model.generate_graphed if graph else model.generate
    gen(prompt[:, :min(prompt_len, 128)], 2)  # warm-up (allocator, first-call set-up)
    toks, t_prefill, t_decode = gen(prompt, gen_len)
    assert toks.shape == (batch, prompt_len + gen_len)
    return {"impl": "b200k" if use_library else "torch", "decode": "cuda graph" if graph else "eager",
            "layers": cfg.n_layers, "batch": batch,
            "prompt_len": prompt_len, "gen_len": gen_len, "prefill_s": t_prefill,
            "prefill_tok_s": batch * prompt_len / t_prefill, "decode_s": t_decode,
            "decode_tok_s": batch * (gen_len - 1) / max(t_decode, 1e-9),
            "total_tok_s": batch * gen_len / (t_prefill + t_decode)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--gen-len", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--baseline", action="store_true", help="also time the torch.matmul / SDPA version")
    ap.add_argument("--no-graph", action="store_true", help="eager decode loop instead of the captured step")
    args = ap.parse_args(argv)
    cfg = LlamaConfig(n_layers=args.layers, n_kv_heads=args.kv_heads)
    print(json.dumps(run(cfg, args.batch, args.prompt_len, args.gen_len, True, graph=not args.no_graph)), flush=True)
    if args.baseline:
        torch.cuda.empty_cache()
        print(json.dumps(run(cfg, args.batch, args.prompt_len, args.gen_len, False, graph=not args.no_graph)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
