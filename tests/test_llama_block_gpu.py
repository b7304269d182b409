"""The Llama-shaped stack built from the library's ops (fused-QKV GEMM, strided causal prefill
attention, split-KV decode over the cache, residual-add and SwiGLU epilogues) against the same stack
on torch.matmul / scaled_dot_product_attention with identical random weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_prefill_and_decode_logits_match_torch_stack(cuda_device, kv_heads):
    from b200k import llama
    cfg = llama.LlamaConfig(hidden=512, n_heads=4, n_kv_heads=kv_heads, head_dim=128, intermediate=1024, n_layers=2,
                            vocab=1024)
    ours = llama.SyntheticLlama(cfg, dtype=torch.float16, use_library=True, seed=3)
    ref = llama.SyntheticLlama(cfg, dtype=torch.float16, use_library=False, seed=3)
    g = torch.Generator(device=cuda_device).manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (3, 200), generator=g, device=cuda_device)
    for m in (ours, ref):
        m.alloc_cache(3, 210)
    with torch.no_grad():
        a, b = ours.forward(prompt, 0), ref.forward(prompt, 0)
        scale = float(b.float().abs().max())
        assert float((a.float() - b.float()).abs().max()) <= 2e-2 * scale
        nxt = b.argmax(-1, keepdim=True)
        for step in range(3):  # decode steps over the cache, same input tokens on both sides
            a, b = ours.forward(nxt, 200 + step), ref.forward(nxt, 200 + step)
            assert float((a.float() - b.float()).abs().max()) <= 2e-2 * scale
            nxt = b.argmax(-1, keepdim=True)


def test_generate_shapes_and_timing(cuda_device):
    from b200k import llama
    cfg = llama.LlamaConfig(hidden=512, n_heads=4, n_kv_heads=4, head_dim=128, intermediate=1024, n_layers=2, vocab=1024)
    out = llama.run(cfg, batch=2, prompt_len=256, gen_len=4, use_library=True, dtype=torch.bfloat16)
    assert out["prefill_tok_s"] > 0 and out["decode_tok_s"] > 0


@pytest.mark.parametrize("use_library", [True, False])
def test_graphed_decode_matches_eager(cuda_device, use_library):
    """The decode step captured in a CUDA graph (device-side position, lengths and token feedback,
    allocation-free decode attention) produces the same greedy tokens as the eager loop."""
    from b200k import llama
    cfg = llama.LlamaConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, intermediate=1024, n_layers=2, vocab=1024)
    model = llama.SyntheticLlama(cfg, dtype=torch.bfloat16, use_library=use_library, seed=5)
    g = torch.Generator(device=cuda_device).manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (3, 150), generator=g, device=cuda_device)
    eager, _, _ = model.generate(prompt, 6)
    graphed, t_prefill, t_decode = model.generate_graphed(prompt, 6)
    assert t_prefill > 0 and t_decode > 0
    if use_library:
        assert torch.equal(eager, graphed)  # same kernels on the same data
    else:
        # the torch comparator's graphed step attends through a mask over the padded cache, the eager
        # one over the sliced cache: different SDPA kernels, so allow rare argmax ties to differ
        assert (eager == graphed).float().mean() > 0.9
