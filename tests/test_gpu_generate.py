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
