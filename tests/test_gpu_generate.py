"""Greedy decode with the decode step captured as a CUDA graph against the same loop run eagerly."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graphed_greedy_decode_equals_eager_loop():
    from latentq_llm_b200 import finetune as ft
    from latentq_llm_b200.generate import GraphedGreedyDecoder
    model = ft.build_model("llama-tiny", "cuda", seed=3)
    ft.quantize_decoder(model, lbit=4, gbit=16)
    model.eval()
    dec = GraphedGreedyDecoder(model, batch=2, max_len=96)
    g = torch.Generator(device="cuda").manual_seed(1)
    for trial in range(2):                                   # the second prompt replays the graph captured for the first
        prompt = torch.randint(0, 1024, (2, 40 + 8 * trial), device="cuda", generator=g)
        eager = dec.generate(prompt, 12, use_graph=False)
        graphed = dec.generate(prompt, 12, use_graph=True)
        assert eager.shape == (2, 12) and torch.equal(eager, graphed), trial
    assert dec.graph is not None
    with pytest.raises(ValueError):
        dec.generate(torch.zeros((2, 90), dtype=torch.long, device="cuda"), 12)


@pytest.mark.parametrize("arch", ["llama-tiny", "llama-gqa-tiny"])
def test_fused_llama_decoder_against_the_eager_modules(arch):
    """The decode step as a chain of this library's kernels (fused q|k|v and gate|up projections, RMSNorm, RoPE with
    the KV-cache write, single-query attention, silu*up) against the model's own eager modules on the same prompt:
    logits of the first decode step agree closely, greedy tokens agree wherever the eager loop's choice was not a
    near-tie, and graph replay equals the eager chain of the same kernels bit for bit."""
    from latentq_llm_b200 import finetune as ft
    from latentq_llm_b200.generate import FusedLlamaGreedyDecoder, GraphedGreedyDecoder, _SDPA
    from torch.nn.attention import sdpa_kernel
    model = ft.build_model(arch, "cuda", seed=3)
    ft.quantize_decoder(model, lbit=4, gbit=16)
    model.eval()
    B, P, T = 2, 40, 10
    fused = FusedLlamaGreedyDecoder(model, batch=B, max_len=96)
    ref = GraphedGreedyDecoder(model, batch=B, max_len=96)
    g = torch.Generator(device="cuda").manual_seed(1)
    prompt = torch.randint(0, 1024, (B, P), device="cuda", generator=g)

    # logits of the first decode step through the eager modules
    ref.cache.reset()
    with torch.no_grad(), sdpa_kernel(_SDPA):
        out = model(input_ids=prompt, past_key_values=ref.cache, cache_position=torch.arange(P, device="cuda"), use_cache=True)
        first = out.logits[:, -1:].argmax(-1)
        out = model(input_ids=first, past_key_values=ref.cache, cache_position=torch.tensor([P], device="cuda"), use_cache=True)
    want_logits = out.logits[:, -1].float()

    toks_eager_chain = fused.generate(prompt, 2, use_graph=False)
    got_logits = fused.logits.float()
    assert torch.equal(toks_eager_chain[:, 0], first.view(-1))
    diff = (got_logits - want_logits).abs().max().item()
    spread = (want_logits.max() - want_logits.min()).item()
    assert diff <= 0.02 * spread, (diff, spread)

    want = ref.generate(prompt, T, use_graph=False)
    got = fused.generate(prompt, T, use_graph=False)
    graphed = fused.generate(prompt, T, use_graph=True)
    assert torch.equal(got, graphed), "graph replay must equal the eager chain of the same kernels"
    agree = (got == want).float().mean().item()
    assert torch.equal(got[:, :2], want[:, :2]) and agree >= 0.7, agree
    # a second prompt replays the captured graph
    prompt2 = torch.randint(0, 1024, (B, P + 8), device="cuda", generator=g)
    assert torch.equal(fused.generate(prompt2, T, use_graph=True), fused.generate(prompt2, T, use_graph=False))


@pytest.mark.parametrize("B", [1, 2])
def test_fused_decoder_with_the_norm_inside_the_projections_decodes_the_same_tokens(monkeypatch, B):
    """One or two sequences at hidden size 4096: the residual add and both RMSNorms of a layer run inside the q|k|v and
    gate|up launches, the residual stream alternating between two buffers.  Same bits as the chain with separate norm
    launches: logits and tokens identical, eager chain and graph replay alike."""
    from latentq_llm_b200 import finetune as ft, ops
    from latentq_llm_b200.generate import FusedLlamaGreedyDecoder
    model = ft.build_model("llama-wide-tiny", "cuda", seed=5)
    ft.quantize_decoder(model, lbit=4, gbit=16)
    model.eval()
    P, T = 24, 8
    g = torch.Generator(device="cuda").manual_seed(B)
    prompt = torch.randint(0, 1024, (B, P), device="cuda", generator=g)
    monkeypatch.setenv("LQ_DECODE_NO_FUSED_NORM", "1")
    plain = FusedLlamaGreedyDecoder(model, batch=B, max_len=64)
    assert not plain.fuse_norm
    want = plain.generate(prompt, T, use_graph=False)
    want_logits = plain.logits.clone()
    monkeypatch.delenv("LQ_DECODE_NO_FUSED_NORM")
    fused = FusedLlamaGreedyDecoder(model, batch=B, max_len=64)
    assert fused.fuse_norm
    calls = []
    real = ops.gemm_a16w4_fwd_rmsnorm
    monkeypatch.setattr(ops, "gemm_a16w4_fwd_rmsnorm", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    got = fused.generate(prompt, T, use_graph=False)
    assert calls and torch.equal(got, want) and torch.equal(fused.logits, want_logits)
    assert torch.equal(fused.generate(prompt, T, use_graph=True), want)
    assert torch.equal(fused.logits, want_logits)
