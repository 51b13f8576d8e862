"""Greedy decode through the quantized model with the per-token work captured as one CUDA graph.

The reference decodes with HF `generate` (generate.py:150-190): every token is a fresh Python walk over the model,
about 230 kernel-launching calls for a 7B Llama, and the GPU waits for the host (decode-sized A16W4 GEMMs run ~10 us
each).  Here the decode step — embedding, all layers with the one-launch decode GEMM (lq_gemv.cu), KV-cache update,
logits, argmax — is captured once on a static KV cache and replayed per token; the token and position live in
device buffers that the captured step itself advances, so a replay needs no host work at all.
"""
from __future__ import annotations

import torch
from torch.nn.attention import SDPBackend, sdpa_kernel

# the cuDNN attention backend rebuilds its plan for every new KV length (milliseconds of host time per layer and token)
_SDPA = [SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]


class GraphedGreedyDecoder:
    """`decoder = GraphedGreedyDecoder(model, batch, max_len)`; `tokens = decoder.generate(prompt, max_new_tokens)`.

    `prompt` is a LongTensor [batch, P] on the model's device with P + max_new_tokens <= max_len.  The first call
    captures the decode step; later calls (any prompt of the same batch size) only replay it."""

    def __init__(self, model, batch: int, max_len: int):
        from transformers import StaticCache
        self.model, self.batch, self.max_len = model, batch, max_len
        self.device = next(model.parameters()).device
        self.cache = StaticCache(config=model.config, max_cache_len=max_len)
        self.tok = torch.zeros((batch, 1), dtype=torch.long, device=self.device)
        self.pos = torch.zeros((1,), dtype=torch.long, device=self.device)
        self.graph = None

    def _step(self):
        out = self.model(input_ids=self.tok, past_key_values=self.cache, cache_position=self.pos, use_cache=True)
        self.tok.copy_(out.logits[:, -1:].argmax(-1))
        self.pos.add_(1)

    @torch.no_grad()
    def _capture(self, tok, pos):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                       # warm-up: lazy initialisations must not be captured
            self.tok.copy_(tok); self.pos.fill_(pos)
            self._step(); self._step()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        self.tok.copy_(tok); self.pos.fill_(pos)
        with torch.cuda.graph(self.graph):
            self._step()
        # cache rows written during warm-up and capture lie at positions >= pos: they are masked until overwritten

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, use_graph: bool = True) -> torch.Tensor:
        b, p = prompt.shape
        if b != self.batch or p + max_new_tokens > self.max_len:
            raise ValueError("prompt does not fit the decoder's batch size / cache length")
        self.model.eval()
        with sdpa_kernel(_SDPA):
            if use_graph and self.graph is None:
                # capture on a throw-away prefill: warm-up and capture advance whatever bookkeeping the cache keeps
                # besides its K/V tensors, so the real decode below starts again from a reset cache
                self.cache.reset()
                out = self.model(input_ids=prompt, past_key_values=self.cache,
                                 cache_position=torch.arange(p, device=self.device), use_cache=True)
                self._capture(out.logits[:, -1:].argmax(-1), p)
            self.cache.reset()
            out = self.model(input_ids=prompt, past_key_values=self.cache,
                             cache_position=torch.arange(p, device=self.device), use_cache=True)
            first = out.logits[:, -1:].argmax(-1)
            self.tok.copy_(first); self.pos.fill_(p)
            toks = [first.clone()]
            for _ in range(max_new_tokens - 1):
                if use_graph:
                    self.graph.replay()
                else:
                    self._step()
                toks.append(self.tok.clone())
        return torch.cat(toks, dim=1)
