"""The reference's generation benchmark driving the library's ops inside a HuggingFace Llama.

What the reference does (benchmarks/huggingface-cuda/hf-gen.py:46-130, benchmarks/utils.py:23-98,
benchmarks/flashattn-cuda/modeling_llama.py:687-690): load a Llama checkpoint in fp16, hang timing
hooks on the model that time the first (prefill) forward between two device synchronisations and then
flip `model.stage` to "decode", call `model.generate(..., max_new_tokens=gen_len, do_sample=False)`,
and derive prefill / decode / total latency and tokens per second; its forked `modeling_llama.py`
sends the attention of every layer to `fmha_unified.ops.fine_fmha(q, k, v, causal=True,
is_decode=False, kernel_index=5)` during prefill and `(..., causal=False, is_decode=True,
kernel_index=5)` during decode.

Here the same flow runs on the installed `transformers` without a fork:
  * `fine_fmha_attention` is registered as the attention implementation "fine_fmha" and makes exactly
    those two calls.  It passes K and V with their own (un-repeated) KV heads: the fork expands them with
    `repeat_kv` first (modeling_llama.py:670-671), which the library's GQA mapping makes unnecessary.
  * `route_linears_through_gemm_unified` sends every projection (q, k, v, o, gate, up, down, lm_head)
    through `gemm_unified.ops.fine_gemm`; the reference leaves them on `nn.Linear` and never calls its
    GEMM package from a model.
  * Checkpoints, tokenizer and prompts are replaced by a randomly initialised model of the same shape
    (weights N(0, 0.02)) and random token ids: nothing here needs the network.
  * The timing hooks, size formulas and log format are the reference's: `harness_utils()` returns the
    reference's own `benchmarks/utils.py` when a checkout is at hand (REFERENCE_ROOT), else the
    equivalents below, which keep its names and argument meaning (tests compare the two).
"""
from __future__ import annotations

import importlib.util
import os
import sys
import time

import torch

GB = 1 << 30


# ------------------------------------------------------------------ mirror of benchmarks/utils.py
def model_bytes(config) -> int:
    """fp16 bytes of a decoder the way benchmarks/utils.py:23-34 counts them: per layer the fused QKV
    and output projections, a 4h MLP (weights and biases) and four norm vectors, plus the embedding."""
    h, layers = config.hidden_size, config.num_hidden_layers
    attention = h * (3 * h + 1) + h * (h + 1)
    mlp = h * (4 * h + 1) + h * 4 * (h + 1)
    norms = h * 4
    embedding = config.vocab_size * (h + 1)
    return 2 * (layers * (attention + mlp + norms) + embedding)


def cache_bytes(config, batch_size: int, seq_len: int) -> int:
    """fp16 bytes of K and V for all layers (benchmarks/utils.py:36-37; it counts full-width heads)."""
    return 2 * batch_size * seq_len * config.num_hidden_layers * config.hidden_size * 2


def write_gen_benchmark_log(model_size, cache_size, gpu_peak_mem, prefill_latency, prefill_throughput,
                            decode_latency, decode_throughput, total_latency, total_throughput) -> str:
    """Same text as benchmarks/utils.py:39-55."""
    rows = [
        (f"model size: {model_size / GB:.3f} GB", f"cache size: {cache_size / GB:.3f} GB",
         f"peak gpu mem: {gpu_peak_mem / GB:.3f} GB"),
        (f"prefill latency: {prefill_latency:.3f} s", f"prefill throughput: {prefill_throughput:.3f} token/s"),
        (f"decode latency: {decode_latency:.3f} s", f"decode throughput: {decode_throughput:.3f} token/s"),
        (f"total latency: {total_latency:.3f} s", f"total throughput: {total_throughput:.3f} token/s"),
    ]
    return "\n".join("\t".join(r) for r in rows)


def add_model_hooks(model: torch.nn.Module) -> None:
    """Forward hooks with the behaviour of benchmarks/utils.py:75-98: while `model.stage == "prefill"`
    the forward is timed between two device synchronisations into `model.__duration__` and the stage
    becomes "decode"; in the decode stage the hooks do nothing."""
    def before(module, args):
        if getattr(module, "stage", None) == "prefill":
            torch.cuda.synchronize()
            module.__start_time__ = time.time()

    def after(module, args, output):
        if getattr(module, "stage", None) == "prefill":
            torch.cuda.synchronize()
            module.__duration__ = time.time() - module.__start_time__
            module.stage = "decode"

    if not hasattr(model, "__start_time_hook_handle__"):
        model.__start_time_hook_handle__ = model.register_forward_pre_hook(before)
    if not hasattr(model, "__end_time_hook_handle__"):
        model.__end_time_hook_handle__ = model.register_forward_hook(after)


def remove_model_hooks(module: torch.nn.Module) -> None:
    """Counterpart of benchmarks/utils.py:101-111."""
    for name in ("__start_time_hook_handle__", "__end_time_hook_handle__"):
        if hasattr(module, name):
            getattr(module, name).remove()
            delattr(module, name)
    for name in ("stage", "__duration__"):
        if hasattr(module, name):
            delattr(module, name)


def load_reference_utils(reference_root: str):
    """The reference's benchmarks/utils.py as a module, imported from a checkout."""
    path = os.path.join(reference_root, "benchmarks", "utils.py")
    spec = importlib.util.spec_from_file_location("reference_benchmarks_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def harness_utils():
    """The reference's own utils module when REFERENCE_ROOT points at a checkout, else this module."""
    root = os.environ.get("REFERENCE_ROOT", "")
    if root and os.path.exists(os.path.join(root, "benchmarks", "utils.py")):
        return load_reference_utils(root)
    return sys.modules[__name__]


# ------------------------------------------------------------------ the ops inside a HF Llama
def fine_fmha_attention(module, query, key, value, attention_mask=None, dropout: float = 0.0, scaling=None,
                        **kwargs):
    """Attention function for transformers' AttentionInterface making the reference's two calls
    (benchmarks/flashattn-cuda/modeling_llama.py:687-690).  query [B,Hq,S,D]; key, value [B,Hkv,Skv,D]
    (cache included, KV heads not repeated).  The stage is read off the shapes: one query row against a
    longer cache is a decode step.  Like the reference's call site it ignores `attention_mask` (no
    padding inside the batch) and uses the 1/sqrt(D) scale.  Returns ([B,S,Hq,D], None)."""
    import fmha_unified
    if query.size(2) == 1 and key.size(2) > 1:
        out = fmha_unified.ops.fine_fmha(query, key, value, causal=False, is_decode=True, kernel_index=5)
    else:
        out = fmha_unified.ops.fine_fmha(query, key, value, causal=True, is_decode=False, kernel_index=5)
    return out.transpose(1, 2), None


def register_attention(name: str = "fine_fmha") -> str:
    from transformers import AttentionInterface
    AttentionInterface.register(name, fine_fmha_attention)
    return name


class FineLinear(torch.nn.Module):
    """y = x W^T of a bias-free nn.Linear through gemm_unified.ops.fine_gemm: the weight is kept as
    [in_features, out_features] (the GEMM's row-major B operand; a one-time transform of the checkpoint
    layout), activations are flattened to [tokens, in_features]."""

    def __init__(self, linear: torch.nn.Linear, kernel_index: int = 12):
        super().__init__()
        if linear.bias is not None:
            raise RuntimeError("FineLinear takes bias-free projections (Llama has no biases)")
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.kernel_index = kernel_index
        self.register_buffer("weight_kn", linear.weight.detach().t().contiguous())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import gemm_unified
        y = gemm_unified.ops.fine_gemm(x.reshape(-1, self.in_features), self.weight_kn, self.kernel_index)
        return y.view(*x.shape[:-1], self.out_features)


def route_linears_through_gemm_unified(model: torch.nn.Module, kernel_index: int = 12) -> int:
    """Replaces every bias-free nn.Linear of the model by FineLinear; returns how many."""
    count = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, torch.nn.Linear) and child.bias is None:
                setattr(parent, name, FineLinear(child, kernel_index))
                count += 1
    return count


LLAMA2_7B = dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                 num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096)


def build_llama(device, dtype=torch.float16, attn_implementation: str = "fine_fmha", route_linears: bool = True,
                seed: int = 0, **config_overrides):
    """A randomly initialised LlamaForCausalLM of the Llama-2-7B shape (or overrides of it), weights
    N(0, 0.02), in fp16 on `device`, with attention and projections routed to the library's ops."""
    from transformers import LlamaConfig, LlamaForCausalLM
    if attn_implementation == "fine_fmha":
        register_attention("fine_fmha")
    cfg = LlamaConfig(**{**LLAMA2_7B, **config_overrides}, attn_implementation=attn_implementation,
                      initializer_range=0.02, tie_word_embeddings=False)
    torch.manual_seed(seed)
    with torch.device(device):
        model = LlamaForCausalLM(cfg).to(dtype)
    model.eval()
    model.generation_config.eos_token_id = None   # random weights: never stop early
    model.generation_config.pad_token_id = 0
    if route_linears:
        route_linears_through_gemm_unified(model)
    return model


def run_generation(model, batch_size: int, prompt_len: int, gen_len: int, trials: int = 3, seed: int = 1,
                   utils=None) -> dict:
    """The measurement loop of benchmarks/huggingface-cuda/hf-gen.py:73-130 on random token ids:
    hooks on, `model.stage = "prefill"`, greedy `generate`, prefill latency from the hook and total
    latency from the wall clock; the same derived numbers and the same log text."""
    utils = utils or harness_utils()
    cfg = model.config
    device = next(model.parameters()).device
    g = torch.Generator().manual_seed(seed)
    input_ids = torch.randint(1, cfg.vocab_size, (batch_size, prompt_len), generator=g).to(device)
    attention_mask = torch.ones_like(input_ids)
    utils.add_model_hooks(model)
    prefill_timings, total_timings = [], []
    output_ids = None
    for _ in range(trials):
        start = time.time()
        with torch.no_grad():
            model.stage = "prefill"
            output_ids = model.generate(input_ids=input_ids, attention_mask=attention_mask,
                                        max_new_tokens=gen_len, min_new_tokens=gen_len, do_sample=False)
            prefill_timings.append(model.__duration__)
        torch.cuda.synchronize()
        total_timings.append(time.time() - start)
    utils.remove_model_hooks(model)
    assert all(len(x) == prompt_len + gen_len for x in output_ids)      # hf-gen.py:100-102
    total_latency, prefill_latency = total_timings[-1], prefill_timings[-1]
    decode_latency = total_latency - prefill_latency
    res = {
        "batch_size": batch_size, "prompt_len": prompt_len, "gen_len": gen_len,
        "prefill_latency": prefill_latency, "prefill_throughput": batch_size * prompt_len / prefill_latency,
        "decode_latency": decode_latency,
        "decode_throughput": batch_size * (gen_len - 1) / max(decode_latency, 1e-10),
        "total_latency": total_latency, "total_throughput": batch_size * gen_len / total_latency,
        "gpu_peak_mem": torch.cuda.max_memory_allocated(device),
        "model_size": utils.model_bytes(cfg), "cache_size": utils.cache_bytes(cfg, batch_size, prompt_len + gen_len),
        "output_ids": output_ids,
    }
    res["log"] = utils.write_gen_benchmark_log(
        res["model_size"], res["cache_size"], res["gpu_peak_mem"], res["prefill_latency"], res["prefill_throughput"],
        res["decode_latency"], res["decode_throughput"], res["total_latency"], res["total_throughput"])
    return res


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="hf-gen style prefill/decode timing on a randomly initialised Llama")
    ap.add_argument("--trials", type=int, default=3)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--prompt_len", type=int, default=512)
    ap.add_argument("--gen_len", type=int, default=32)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--kv_heads", type=int, default=32)
    ap.add_argument("--stock", action="store_true", help="stock transformers path (sdpa attention, nn.Linear)")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    model = build_llama(dev, attn_implementation="sdpa" if args.stock else "fine_fmha",
                        route_linears=not args.stock, num_hidden_layers=args.layers, num_key_value_heads=args.kv_heads)
    res = run_generation(model, args.batch_size, args.prompt_len, args.gen_len, args.trials)
    print(("stock transformers" if args.stock else "library ops") + f", {args.layers} layers")
    print(res["log"])
    return 0


if __name__ == "__main__":
    sys.exit(main())
