"""The reference's generation benchmark flow (benchmarks/huggingface-cuda/hf-gen.py:73-130 with the
timing hooks of benchmarks/utils.py:75-98) on a randomly initialised 2-layer HuggingFace Llama whose
attention makes the reference's two fine_fmha calls (benchmarks/flashattn-cuda/modeling_llama.py:687-690)
and whose projections go through gemm_unified: results agree with the stock transformers path (sdpa
attention, nn.Linear) on the same weights, and the harness reports the reference's numbers."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SMALL = dict(hidden_size=1024, intermediate_size=2816, num_hidden_layers=2, num_attention_heads=8,
             vocab_size=2048, max_position_embeddings=1024)


@pytest.mark.parametrize("kv_heads", [8, 2])
def test_routed_llama_matches_stock_transformers(cuda_device, kv_heads):
    from b200k import _lib, hf_harness
    routed = hf_harness.build_llama(cuda_device, seed=3, num_key_value_heads=kv_heads, **SMALL)
    stock = hf_harness.build_llama(cuda_device, attn_implementation="sdpa", route_linears=False, seed=3,
                                   num_key_value_heads=kv_heads, **SMALL)
    assert routed.config._attn_implementation == "fine_fmha"
    assert sum(isinstance(m, hf_harness.FineLinear) for m in routed.modules()) == 2 * 7 + 1
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(1, SMALL["vocab_size"], (3, 70), generator=g).to(cuda_device)
    n0 = _lib.launch_count()
    with torch.no_grad():
        a = routed(input_ids=ids).logits.float()
        b = stock(input_ids=ids).logits.float()
    assert _lib.launch_count() - n0 >= 2 * 8 + 1   # 7 projections + attention per layer, and the head
    assert float((a - b).abs().max()) <= 2e-2 * max(1.0, float(b.abs().max()))
    # greedy decoding through the cache: prefill + decode calls; compare the tokens where the stock
    # model's choice is not a near-tie (random weights give nearly flat logits now and then)
    with torch.no_grad():
        out_r = routed.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=6,
                                min_new_tokens=6, do_sample=False)
        out_s = stock.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=6,
                               min_new_tokens=6, do_sample=False)
    assert out_r.shape == out_s.shape == (3, 76)
    assert torch.equal(out_r[:, :70], ids)
    assert (out_r[:, 70] == out_s[:, 70]).float().mean() >= 2 / 3


def test_generation_benchmark_flow(cuda_device):
    from b200k import _lib, hf_harness
    model = hf_harness.build_llama(cuda_device, seed=1, num_key_value_heads=2, **SMALL)
    n0 = _lib.launch_count()
    res = hf_harness.run_generation(model, batch_size=4, prompt_len=96, gen_len=8, trials=2, utils=hf_harness)
    launches = _lib.launch_count() - n0
    # per trial: 1 prefill forward and 7 decode forwards, each 2 layers x (7 GEMMs + attention) + head
    assert launches >= 2 * 8 * (2 * 8 + 1)
    assert res["output_ids"].shape == (4, 104)
    assert 0 < res["prefill_latency"] < res["total_latency"]
    assert res["prefill_throughput"] == pytest.approx(4 * 96 / res["prefill_latency"])
    assert res["decode_throughput"] == pytest.approx(4 * 7 / res["decode_latency"])
    assert res["model_size"] == hf_harness.model_bytes(model.config)
    assert res["cache_size"] == hf_harness.cache_bytes(model.config, 4, 104)
    for field in ("model size", "prefill latency", "prefill throughput", "decode throughput", "total latency"):
        assert field in res["log"]
    assert not hasattr(model, "stage") and len(model._forward_hooks) == 0
