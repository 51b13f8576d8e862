"""Greedy decode through the quantized model with the per-token work captured as one CUDA graph.

The reference decodes with HF `generate` (generate.py:150-190): every token is a fresh Python walk over the model,
about 230 kernel-launching calls for a 7B Llama, and the GPU waits for the host (decode-sized A16W4 GEMMs run ~10 us
each).  Here the decode step — embedding, all layers with the one-launch decode GEMM (lq_gemv.cu), KV-cache update,
logits, argmax — is captured once on a static KV cache and replayed per token; the token and position live in
device buffers that the captured step itself advances, so a replay needs no host work at all.
"""
from __future__ import annotations

import os

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
        from . import ops
        with ops.decode_chain():          # the decode-sized GEMMs may fetch their (constant) weights while their predecessor runs
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


class FusedLlamaGreedyDecoder:
    """Greedy decode of a Llama-architecture model (RMSNorm / RoPE / SwiGLU, no biases) whose decoder linears are
    `QLinearA16W4`, with the decode step written as a chain of this library's kernels instead of the eager modules:

        per layer   residual add + RMSNorm -> fused q|k|v projection (one launch, N = (Hq + 2 Hkv) hd) -> RoPE on q, k
                    with k, v written into the KV cache -> single-query attention over the cache -> o projection ->
                    residual add + RMSNorm -> fused gate|up projection (N = 2 I) -> silu(gate) * up -> down projection
        then        residual add + final RMSNorm -> lm_head -> argmax -> embedding of the new token

    eight launches per layer at decode-sized batches, where silu(gate) * up is the epilogue of the gate|up launch, nine
    otherwise (the reference's fusion list: PTQ/quant/fused_attn.py:164-204 fused QKV, :8-58 RoPE,
    PTQ/quant/fused_mlp.py:84-168 gate/up with the silu epilogue, PTQ/quant/triton_norm.py:7-39 RMSNorm), captured
    once as a CUDA graph and replayed per token.  The prompt is prefilled through the model's own modules into the
    same static KV cache.  `hf_rounding=True` rounds intermediates like the eager modules' bf16 tensor ops."""

    def __init__(self, model, batch: int, max_len: int, hf_rounding: bool = True):
        from transformers import StaticCache
        from .quant import QLinearA16W4
        cfg = model.config
        self.model, self.batch, self.max_len, self.hf = model, batch, max_len, hf_rounding
        self.device = dev = next(model.parameters()).device
        self.Hq, self.Hkv = cfg.num_attention_heads, getattr(cfg, "num_key_value_heads", None) or cfg.num_attention_heads
        self.hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.D, self.I, self.eps = cfg.hidden_size, cfg.intermediate_size, cfg.rms_norm_eps
        self.inv_freq = model.model.rotary_emb.inv_freq.detach().to(dev, torch.float32).contiguous()
        self.cache = StaticCache(config=cfg, max_cache_len=max_len)

        def flat(lin):
            if not isinstance(lin, QLinearA16W4) or lin.bias is not None:
                raise TypeError("FusedLlamaGreedyDecoder needs bias-free QLinearA16W4 projections")
            sc, zr, _ = lin.weight.qparam
            return lin.weight.data.reshape(-1), sc.reshape(-1), zr.reshape(-1)

        def fuse(*lins):
            parts = [flat(l) for l in lins]
            return tuple(torch.cat([p[i] for p in parts]).contiguous() for i in range(3))

        self.layers = []
        for layer in model.model.layers:
            a, m = layer.self_attn, layer.mlp
            self.layers.append(dict(ln1=layer.input_layernorm.weight.detach(), ln2=layer.post_attention_layernorm.weight.detach(),
                                    qkv=fuse(a.q_proj, a.k_proj, a.v_proj), o=flat(a.o_proj),
                                    gu=fuse(m.gate_proj, m.up_proj), down=flat(m.down_proj)))
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.h = torch.zeros((batch, self.D), **bf)
        self.xn = torch.zeros((batch, self.D), **bf)
        self.qkv = torch.zeros((batch, (self.Hq + 2 * self.Hkv) * self.hd), **bf)
        self.att = torch.zeros((batch, self.Hq * self.hd), **bf)
        self.tmp = torch.zeros((batch, self.D), **bf)
        self.h2 = torch.zeros((batch, self.D), **bf)
        self.fuse_norm = batch <= 2 and not os.environ.get("LQ_DECODE_NO_FUSED_NORM")
        self.fuse_rope = batch <= 16 and not os.environ.get("LQ_DECODE_NO_FUSED_ROPE")
        self.gu = torch.zeros((batch, 2 * self.I), **bf)
        self.act = torch.zeros((batch, self.I), **bf)
        self.tok = torch.zeros((batch,), dtype=torch.long, device=dev)
        self.pos = torch.zeros((batch,), dtype=torch.long, device=dev)
        self.logits = None
        self.graph = None

    def _step(self):
        from . import ops
        with ops.decode_chain():          # launches may start while their predecessor runs (weights are constant here)
            self._step_kernels(ops)

    def _qkv(self, ops, L, h, h_alt, delta, kc, vc) -> bool:
        """Residual add + RMSNorm + q|k|v projection + RoPE + cache write of one layer in as few launches as the batch
        allows: one (one or two sequences at hidden size 4096), two (up to 16 sequences: RoPE and the cache write are
        the projection's epilogue) or three.  True when the residual stream now lives in `h_alt`."""
        Hq, Hkv, hd, D = self.Hq, self.Hkv, self.hd, self.D
        N = (Hq + 2 * Hkv) * hd
        rope = (self.pos, self.inv_freq, kc, vc, Hq, Hkv, hd, D)
        kw = dict(out=self.qkv, hf_rounding=self.hf)
        norm = (h, delta, L["ln1"], self.eps, h_alt)
        if self.fuse_norm and self.fuse_rope and ops.gemm_a16w4_fwd_qkv_rope(None, *L["qkv"], *rope, norm=norm, **kw) is not None:
            return delta is not None
        if self.fuse_norm and ops.gemm_a16w4_fwd_rmsnorm(*norm, *L["qkv"], N, D, **kw) is not None:
            ops.rope_kv_store(self.qkv, self.pos, self.inv_freq, kc, vc, Hq, Hkv, hd, hf_rounding=self.hf)
            return delta is not None
        ops.add_rmsnorm(h, delta, L["ln1"], self.eps, out=self.xn, hf_rounding=self.hf)
        if not (self.fuse_rope and ops.gemm_a16w4_fwd_qkv_rope(self.xn, *L["qkv"], *rope, **kw) is not None):
            ops.gemm_a16w4_fwd(self.xn, *L["qkv"], None, N, D, out=self.qkv)
            ops.rope_kv_store(self.qkv, self.pos, self.inv_freq, kc, vc, Hq, Hkv, hd, hf_rounding=self.hf)
        return False

    def _step_kernels(self, ops):
        D, I, Hq, Hkv, hd = self.D, self.I, self.Hq, self.Hkv, self.hd
        delta = None                        # self.h holds the embedding row of self.tok (written by the previous step's end)
        h, h_alt = self.h, self.h2          # the residual stream alternates between two buffers where the norm is fused
        for li, L in enumerate(self.layers):
            kc, vc = self.cache.layers[li].keys, self.cache.layers[li].values
            if self._qkv(ops, L, h, h_alt, delta, kc, vc):
                h, h_alt = h_alt, h
            ops.decode_attention(self.qkv, self.pos, kc, vc, Hq, Hkv, hd, out=self.att)
            ops.gemm_a16w4_fwd(self.att, *L["o"], None, D, Hq * hd, out=self.tmp)
            fused = self.fuse_norm and ops.gemm_a16w4_fwd_rmsnorm(h, self.tmp, L["ln2"], self.eps, h_alt, *L["gu"], 2 * I, D,
                                                                 out=self.act, silu_pair=True, hf_rounding=self.hf)
            if fused is None or fused is False:
                ops.add_rmsnorm(h, self.tmp, L["ln2"], self.eps, out=self.xn, hf_rounding=self.hf)
                ops.gemm_a16w4_fwd_silu(self.xn, *L["gu"], I, D, out=self.act, gate_up=self.gu, hf_rounding=self.hf)
            else:
                h, h_alt = h_alt, h
            ops.gemm_a16w4_fwd(self.act, *L["down"], None, D, I, out=self.tmp)
            delta = self.tmp
        ops.add_rmsnorm(h, delta, self.model.model.norm.weight.detach(), self.eps, out=self.xn, hf_rounding=self.hf)
        self.logits = torch.nn.functional.linear(self.xn, self.model.lm_head.weight)
        # argmax, position += 1 and the next step's embedding row in one launch
        ops.argmax_embed(self.logits, self.tok, self.pos, self.model.model.embed_tokens.weight.detach(), self.h)

    def _seed(self, first, p):
        self.tok.copy_(first); self.pos.fill_(p)
        self.h.copy_(torch.nn.functional.embedding(self.tok, self.model.model.embed_tokens.weight))

    @torch.no_grad()
    def _prefill(self, prompt):
        p = prompt.shape[1]
        self.cache.reset()
        with sdpa_kernel(_SDPA):
            out = self.model(input_ids=prompt, past_key_values=self.cache,
                             cache_position=torch.arange(p, device=self.device), use_cache=True)
        return out.logits[:, -1].argmax(-1)

    @torch.no_grad()
    def _capture(self, first, p):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                       # warm-up: lazy initialisations must not be captured
            self._seed(first, p)
            self._step(); self._step()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        self._seed(first, p)
        with torch.cuda.graph(self.graph):
            self._step()

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, use_graph: bool = True) -> torch.Tensor:
        b, p = prompt.shape
        if b != self.batch or p + max_new_tokens > self.max_len:
            raise ValueError("prompt does not fit the decoder's batch size / cache length")
        self.model.eval()
        if use_graph and self.graph is None:
            self._capture(self._prefill(prompt), p)         # throw-away prefill: capture needs an initialised cache
        first = self._prefill(prompt)
        self._seed(first, p)
        toks = [first.clone()]
        for _ in range(max_new_tokens - 1):
            if use_graph:
                self.graph.replay()
            else:
                self._step()
            toks.append(self.tok.clone())
        return torch.stack(toks, dim=1)
