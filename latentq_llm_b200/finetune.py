"""DeepSpeed-free latent fine-tune step around the quantized hot path (the loop of main0.py:526-544).

What it reproduces from the reference driver: every `nn.Linear` inside the decoder layers becomes a
`QLinearA16W4` (main0.py:299-343), every such module gets the backward hook (main0.py:454-461), the
optimizer is `MyAdam(betas=(0.9, 0.95))` over [quantized weights] + [biases and other weights of the decoder
layers] (main0.py:445-472), the loss of each micro-batch is divided by the accumulation count and the
optimizer steps at the accumulation boundary (main0.py:538-543; DeepSpeed does the same internally).
What is new: data parallelism that really covers the quantized weights — their bf16 gradients accumulate in
one flat arena that is all-reduced once per optimizer step (see dp.py).

No datasets or checkpoints are involved: models are built from a config with random weights, quantized with
the reference's min/max rule (PTQ/quant/quantizer.py:34-74) on group-128 slices, and fed uniform random
token ids.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from .dp import ChunkReducer, GradArena, StepGate, allreduce_mean, shard_micro_batches
from .quant import GROUPSIZE, MyAdam, QLinearA16W4

ARCHS = {
    # OPT-1.3B: 24 layers, d 2048, ffn 8192, 32 heads, vocab 50272
    "opt-1.3b": dict(kind="opt", hidden_size=2048, ffn_dim=8192, num_hidden_layers=24, num_attention_heads=32,
                     vocab_size=50272, max_position_embeddings=2048, word_embed_proj_dim=2048),
    # Llama-2-7B: 32 layers, d 4096, ffn 11008, 32 heads, vocab 32000
    "llama-2-7b": dict(kind="llama", hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096),
    # small shapes of the same architectures for tests
    "opt-tiny": dict(kind="opt", hidden_size=256, ffn_dim=512, num_hidden_layers=2, num_attention_heads=4,
                     vocab_size=1024, max_position_embeddings=256, word_embed_proj_dim=256),
    "llama-tiny": dict(kind="llama", hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=4, vocab_size=1024, max_position_embeddings=256),
    # grouped KV heads (8 query heads on 2 KV heads, head size 64)
    "llama-gqa-tiny": dict(kind="llama", hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                           num_key_value_heads=2, vocab_size=1024, max_position_embeddings=256),
    # the 7B hidden size (the decode kernels' written-out K = 4096 paths) with two thin layers
    "llama-wide-tiny": dict(kind="llama", hidden_size=4096, intermediate_size=1024, num_hidden_layers=2,
                            num_attention_heads=32, num_key_value_heads=32, vocab_size=1024, max_position_embeddings=256),
}


def build_model(arch: str, device="cuda", seed: int = 1234, layers: int | None = None) -> nn.Module:
    """Random-init HF model of the named architecture in bf16 (no download: config only)."""
    cfg = dict(ARCHS[arch])
    kind = cfg.pop("kind")
    if layers is not None:
        cfg["num_hidden_layers"] = layers
    torch.manual_seed(seed)
    # parameters are created and initialised on the target device (a 7B model takes minutes to initialise on the host)
    with torch.device(device):
        if kind == "opt":
            from transformers import OPTConfig, OPTForCausalLM
            model = OPTForCausalLM(OPTConfig(**cfg, torch_dtype=torch.bfloat16))
        else:
            from transformers import LlamaConfig, LlamaForCausalLM
            model = LlamaForCausalLM(LlamaConfig(**cfg, torch_dtype=torch.bfloat16))
    return model.to(torch.bfloat16).to(device)


def decoder_layers(model: nn.Module):
    inner = model.model
    return inner.decoder.layers if hasattr(inner, "decoder") else inner.layers


@torch.no_grad()
def quantize_decoder(model: nn.Module, lbit: int = 4, gbit: int = 16) -> list:
    """Swap every nn.Linear inside the decoder layers for a QLinearA16W4 holding int4 group-128 codes of the
    same weights (main0.py:299-343 with the checkpoint replaced by on-the-fly min/max quantization)."""
    swapped = []
    for li, layer in enumerate(decoder_layers(model)):
        for subname, sub in list(layer.named_modules()):
            for name, child in list(sub.named_children()):
                if not isinstance(child, nn.Linear):
                    continue
                n_out, n_in = child.weight.shape
                new = QLinearA16W4(n_in, n_out, bias=child.bias is not None, lbit=lbit, gbit=gbit)
                w = child.weight.data.to(torch.bfloat16).contiguous()
                s, z = ops.find_qparams(w, GROUPSIZE, 15, False)
                new.scales.data = s.view(-1, 1).to(torch.bfloat16)
                new.zeros.data = z.view(-1, 1).to(torch.bfloat16)
                codes, _ = ops.a16w4_requant(w, new.scales.data.view(-1), new.zeros.data.view(-1),
                                             ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16))
                new.weight.set_value(codes, [new.scales, new.zeros, new.wshape])
                new.lname = f"layers.{li}.{subname + '.' if subname else ''}{name}"
                if lbit == 4:
                    new.weight.residual.name = new.lname + ".residual"
                if child.bias is not None:
                    new.bias.data = child.bias.data.to(torch.bfloat16)
                new.to(w.device)
                setattr(sub, name, new)
                swapped.append(new)
    return swapped


def build_optimizer(model: nn.Module, lr: float = 1e-3, obit: int = 8, mu_f: int = 20, direct_grad: bool = True):
    """Parameter groups of main0.py:445-472: [quantized weights], [biases + other decoder-layer weights]."""
    for p in model.parameters():
        p.requires_grad_(False)
    groups = [{"params": [], "weight_decay": 0.0}, {"params": [], "weight_decay": 0.0}]
    for layer in decoder_layers(model):
        for child in layer.modules():
            if getattr(child, "bias", None) is not None and isinstance(child.bias, torch.Tensor):
                child.bias.requires_grad_(True)
                groups[1]["params"].append(child.bias)
            if isinstance(child, QLinearA16W4):
                child.weight.requires_grad = True
                child.add_hook(direct=direct_grad)     # False: the reference's backward-hook route
                groups[0]["params"].append(child.weight)
            elif isinstance(getattr(child, "weight", None), nn.Parameter) and not isinstance(child, nn.Embedding):
                child.weight.requires_grad_(True)
                groups[1]["params"].append(child.weight)
    opt = MyAdam(groups, lr=lr, betas=(0.9, 0.95), obit=obit, mu_updata_f=mu_f)
    return opt, groups


class LatentFineTuner:
    """One optimizer step = `grad_accum` micro-batches of forward/backward on this rank, one mean all-reduce of the
    gradient arena (by runs of layers, overlapped with the last backward pass and the optimizer step), one MyAdam step
    (dequantize + Adam + stochastic requantize per quantized weight)."""

    def __init__(self, model, optimizer, groups, grad_accum: int = 8, group=None, gate_timeout_s: float = 600.0,
                 cuda_graph: bool = False, overlap_chunks: int = 8, run_id: str = "0"):
        """`cuda_graph=True`: forward + backward of one micro-batch are captured once (first `step`, fixed [B, S]) and
        replayed; the ~430 kernel-launching Python calls per micro-batch (144 quantized linears, three GEMMs each)
        otherwise leave the GPU waiting for the host.

        `overlap_chunks` (world size > 1): the decoder layers are cut into that many runs; during the backward pass of
        the step's last micro-batch the gradients of a run are all-reduced as soon as the pass has left the run (its
        layers come last in the forward order, first in the backward order), and the optimizer then steps run by run
        as the reductions land.  0 = one bucketed all-reduce after the backward pass.

        `run_id` names this launch of the job in the step gate's keys (give a restarted job a new one)."""
        self.model, self.opt, self.grad_accum, self.group = model, optimizer, grad_accum, group
        self.cuda_graph, self._graph, self._static_ids, self._static_loss, self._graph_scale = cuda_graph, None, None, None, None
        self.params = groups[0]["params"] + groups[1]["params"]
        self.arena = GradArena(self.params, dtype=torch.bfloat16, device=next(model.parameters()).device)
        self.step_no = 0
        self.exchange = True                    # False: skip the gradient exchange (timing the step without it)
        dist_on = torch.distributed.is_available() and torch.distributed.is_initialized()
        self.gate = StepGate(timeout_s=gate_timeout_s, nonce=run_id) if dist_on and torch.distributed.get_world_size() > 1 else None
        self._reducer, self._events, self._capturing, self._reduce_in_backward = None, {}, False, False
        if self.gate is not None and overlap_chunks > 0:
            self._plan_overlap(groups, overlap_chunks)
        # the hidden states entering the first decoder layer must require grad, otherwise autograd skips the custom
        # backward of the quantized linears (embeddings are frozen, as in the reference's parameter groups)
        model.get_input_embeddings().register_forward_hook(lambda m, i, o: o.requires_grad_(True))

    def step(self, micro_batches) -> torch.Tensor:
        """`micro_batches`: list of LongTensor [B, S] of token ids for THIS rank.  Returns the mean loss (device tensor)."""
        self.model.train()
        self.arena.attach()
        total = torch.zeros((), device=self.arena.flat.device, dtype=torch.float32)
        if self.cuda_graph:
            self._ensure_graph(micro_batches[0], len(micro_batches))
        red, last = (self._reducer if self.exchange else None), len(micro_batches) - 1
        for i, ids in enumerate(micro_batches):
            if red is not None and i == last:
                self.gate.arrive_and_wait(self.step_no)  # host-side liveness check before the step's first collective
                red.begin()
                self._reduce_in_backward = not self.cuda_graph
            if self.cuda_graph:
                self._static_ids.copy_(ids, non_blocking=True)
                self._graph.replay()
                total += self._static_loss.detach().float()
                if red is not None and i == last:        # the replayed backward pass records one event per run of layers
                    for k in sorted(self._events, reverse=True):
                        red.launch(k, after_event=self._events[k])
                continue
            out = self.model(input_ids=ids, labels=ids, use_cache=False)
            (out.loss / len(micro_batches)).backward()   # (last micro-batch: the layer hooks launch the reductions)
            total += out.loss.detach().float()
        self._reduce_in_backward = False
        if red is not None:
            for k in range(len(red.ranges)):             # whatever is left: the first run of layers, the dense parameters
                red.launch(k)
            self.opt.before_param = self._wait_for_param
            self.opt.last_to_first = True                # the order the reductions were queued in: last run first
            self.opt.step()
            red.wait_all()
        else:
            if self.gate is not None and self.exchange:
                self.gate.arrive_and_wait(self.step_no)  # host-side liveness check before the collective
                allreduce_mean(self.arena, self.group)
            self.opt.step()
        for p in self.params:                           # MyAdam drops quantized grads (p.grad = None); clear the rest too
            p.grad = None
        self.step_no += 1
        return total / max(1, len(micro_batches))


    def _plan_overlap(self, groups, n_chunks: int) -> None:
        """Cut the quantized-weight part of the arena into runs of consecutive decoder layers; the dense parameters
        (biases, norms: a few MB) form one more range, reduced after the backward pass."""
        layers = list(decoder_layers(self.model))
        layer_of = {}
        for li, layer in enumerate(layers):
            for child in layer.modules():
                if isinstance(child, QLinearA16W4):
                    layer_of[id(child.weight)] = li
        qp = groups[0]["params"]
        order = [layer_of.get(id(p), -1) for p in qp]
        if not qp or min(order) < 0 or any(b < a for a, b in zip(order, order[1:])):
            return                                        # parameters not in layer order: keep the single all-reduce
        q_end = self.arena.offsets[len(qp)] if len(self.params) > len(qp) else self.arena.numel
        n_chunks = max(1, min(n_chunks, len(layers)))
        first_layer = [round(k * len(layers) / n_chunks) for k in range(n_chunks)]
        starts = []
        for fl in first_layer:                            # arena offset of the first quantized weight of layer >= fl
            idx = next((i for i, l in enumerate(order) if l >= fl), None)
            starts.append(q_end if idx is None else self.arena.offsets[idx])
        ranges = [(starts[k], starts[k + 1] if k + 1 < n_chunks else q_end) for k in range(n_chunks)]
        ranges.append((q_end, self.arena.numel))
        self._reducer = ChunkReducer(self.arena, ranges, self.group)
        self._range_of = {}
        for i, p in enumerate(self.params):
            off = self.arena.offsets[i]
            self._range_of[id(p)] = next(k for k, (a, b) in enumerate(ranges) if a <= off < b or (a == b == off))
        for k in range(1, n_chunks):                      # run k is final once the backward pass enters the layer below it
            if ranges[k][1] > ranges[k][0]:
                layers[first_layer[k] - 1].register_full_backward_pre_hook(lambda m, go, k=k: self._run_done(k))
                self._events[k] = None

    def _run_done(self, k: int) -> None:
        if self._capturing:
            if self._events.get(k) is None:
                # external: the captured record becomes an event node that streams outside the graph can wait for
                self._events[k] = torch.cuda.Event(external=True)
            self._events[k].record()
        elif self._reduce_in_backward:
            self._reducer.launch(k)

    def _wait_for_param(self, p) -> None:
        self._reducer.wait(self._range_of[id(p)])

    def _ensure_graph(self, ids, n_micro):
        """Capture forward + backward of one micro-batch (gradients accumulate in place in the arena views)."""
        if self._graph is not None:
            if tuple(ids.shape) != tuple(self._static_ids.shape) or n_micro != self._graph_scale:
                raise ValueError("the captured step has a fixed micro-batch shape and accumulation count")
            return
        self._static_ids = ids.clone()
        self._graph_scale = n_micro
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                         # warm-up on a side stream: lazy initialisations, autograd buffers
            for _ in range(2):
                out = self.model(input_ids=self._static_ids, labels=self._static_ids, use_cache=False)
                (out.loss / n_micro).backward()
        torch.cuda.current_stream().wait_stream(side)
        self._graph = torch.cuda.CUDAGraph()
        self._capturing = True
        quiet = getattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch", None)
        if quiet is not None:
            quiet(False)            # warm-up (side stream) and capture (capture stream) differ on purpose
        try:
            with torch.cuda.graph(self._graph):
                out = self.model(input_ids=self._static_ids, labels=self._static_ids, use_cache=False)
                self._static_loss = out.loss
                (out.loss / n_micro).backward()
        finally:
            self._capturing = False
        self.arena.attach()                                   # drop what warm-up and capture accumulated


def synthetic_batches(n: int, batch: int, seq: int, vocab: int, device, seed: int):
    g = torch.Generator(device=device).manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), device=device, generator=g) for _ in range(n)]


# ---------------------------------------------------------------------------------------------------
# Checkpoint I/O in the reference's key layout (main0.py:299-343 reads `<decoder>.<i>.<sub>.{qweight,zeros,scales,bias}`)
# ---------------------------------------------------------------------------------------------------
def decoder_prefix(model: nn.Module) -> str:
    return "model.decoder.layers." if hasattr(model.model, "decoder") else "model.layers."


@torch.no_grad()
def save_quantized_decoder(model: nn.Module, path: str, with_residual: bool = True) -> int:
    """Write every QLinearA16W4 of the decoder as the reference's A16W4 checkpoint keys: `qweight` int8 nibble pairs
    (flat, the layout the GEMMs read), `zeros` / `scales` [G, 1], `bias`.  With `with_residual` the 4-bit residual words
    and the curve level travel too (`residual_int`, `residual_mu`: an extension, needed to resume training exactly).
    Returns the number of layers written."""
    from safetensors.torch import save_file
    prefix, out, n = decoder_prefix(model), {}, 0
    for li, layer in enumerate(decoder_layers(model)):
        for subname, sub in layer.named_modules():
            if not isinstance(sub, QLinearA16W4):
                continue
            key = f"{prefix}{li}.{subname}"
            out[key + ".qweight"] = sub.weight.data.reshape(-1).contiguous().cpu()
            out[key + ".zeros"] = sub.zeros.data.contiguous().cpu()
            out[key + ".scales"] = sub.scales.data.contiguous().cpu()
            if sub.bias is not None:
                out[key + ".bias"] = sub.bias.data.contiguous().cpu()
            res = getattr(sub.weight, "residual", None)
            if with_residual and res is not None and hasattr(res, "residual_int") and not res.init:
                out[key + ".residual_int"] = res.residual_int.reshape(-1).contiguous().cpu()
                out[key + ".residual_mu"] = torch.tensor([res.mu, res.lock_mu], dtype=torch.int32)
            n += 1
    save_file(out, path)
    return n


@torch.no_grad()
def load_quantized_decoder(model: nn.Module, ckt, lbit: int = 4, gbit: int = 16) -> list:
    """The A16W4 branch of main0.py:299-343: swap every nn.Linear of the decoder layers for a QLinearA16W4 filled from the
    checkpoint (`ckt`: a path to a .safetensors file or a dict of tensors with the keys above)."""
    if isinstance(ckt, str):
        from safetensors.torch import load_file
        ckt = load_file(ckt)
    prefix, swapped = decoder_prefix(model), []
    for li, layer in enumerate(decoder_layers(model)):
        for subname, sub in list(layer.named_modules()):
            for name, child in list(sub.named_children()):
                if not isinstance(child, (nn.Linear, QLinearA16W4)):
                    continue
                qual = f"{subname + '.' if subname else ''}{name}"
                key = f"{prefix}{li}.{qual}"
                dev = child.weight.data.device if isinstance(child, nn.Linear) else child.scales.device
                n_out, n_in = (child.weight.shape if isinstance(child, nn.Linear) else child.wshape)
                new = QLinearA16W4(int(n_in), int(n_out), bias=child.bias is not None, lbit=lbit, gbit=gbit)
                new.lname = key
                new.zeros.data = ckt[key + ".zeros"].to(torch.bfloat16).to(dev)
                new.scales.data = ckt[key + ".scales"].to(torch.bfloat16).to(dev)
                new.weight.set_value(ckt[key + ".qweight"].to(dev), [new.scales, new.zeros, new.wshape])
                if lbit == 4:
                    new.weight.residual.name = key + ".residual"
                    if key + ".residual_int" in ckt:
                        res = new.weight.residual
                        res.residual_int.copy_(ckt[key + ".residual_int"].to(dev).view_as(res.residual_int))
                        mu, lock_mu = (int(v) for v in ckt[key + ".residual_mu"].tolist())
                        res.mu = lock_mu                           # _after_set_value copies mu into lock_mu
                        res._after_set_value(new.scales.data.view(-1, 1))
                        res.mu = mu
                if child.bias is not None:
                    new.bias.data = ckt[key + ".bias"].to(torch.bfloat16).to(dev)
                new.to(dev)
                setattr(sub, name, new)
                swapped.append(new)
    return swapped


# ---------------------------------------------------------------------------------------------------
# Exact resume: everything the next optimizer step reads (the reference saves the model only, main0.py:585-588)
# ---------------------------------------------------------------------------------------------------
_STATE_KEYS = ("state1", "state2", "qmap1", "absmax1", "qmap2", "absmax2")


@torch.no_grad()
def save_training_state(model: nn.Module, optimizer: MyAdam, groups, path: str, step_no: int = 0) -> int:
    """One .safetensors file with, per trained parameter in optimizer order (`<group>.<index>`): packed codes, residual
    words and curve levels of a quantized weight, or the dense tensor; both optimizer states with their block parameters
    and the step count.  Quantization parameters (`scales`, `zeros`) are frozen and travel with the model checkpoint
    (`save_quantized_decoder`).  Returns the number of tensors written."""
    from safetensors.torch import save_file
    from .quant import QuantTensor
    out = {"meta.step_no": torch.tensor([int(step_no)], dtype=torch.int64)}
    for gi, group in enumerate(groups):
        for pi, p in enumerate(group["params"]):
            key = f"{gi}.{pi}"
            if isinstance(p, QuantTensor):
                out[key + ".codes"] = p.data.reshape(-1).contiguous().cpu()
                res = getattr(p, "residual", None)
                if res is not None and hasattr(res, "residual_int"):
                    out[key + ".residual_int"] = res.residual_int.reshape(-1).contiguous().cpu()
                    out[key + ".residual_meta"] = torch.tensor([res.mu, res.lock_mu, int(res.init)], dtype=torch.int32)
            else:
                out[key + ".dense"] = p.data.contiguous().cpu()
            st = optimizer.state.get(p, {})
            if len(st):
                out[key + ".opt_step"] = torch.tensor([int(st["step"])], dtype=torch.int64)
                for k in _STATE_KEYS:
                    if k in st:
                        out[f"{key}.opt_{k}"] = st[k].contiguous().cpu()
    save_file(out, path)
    return len(out)


@torch.no_grad()
def load_training_state(model: nn.Module, optimizer: MyAdam, groups, ckt) -> int:
    """Restore `save_training_state` into a model / optimizer of the same structure, IN PLACE (parameter objects, gradient
    arena views and a captured CUDA graph stay valid).  Returns the saved step number."""
    if isinstance(ckt, str):
        from safetensors.torch import load_file
        ckt = load_file(ckt)
    from .quant import QuantTensor
    for gi, group in enumerate(groups):
        for pi, p in enumerate(group["params"]):
            key = f"{gi}.{pi}"
            if isinstance(p, QuantTensor):
                p.data.view(-1).copy_(ckt[key + ".codes"].to(p.data.device).view(p.data.dtype))
                res = getattr(p, "residual", None)
                if res is not None and key + ".residual_int" in ckt:
                    res.residual_int.view(-1).copy_(ckt[key + ".residual_int"].to(res.residual_int.device))
                    mu, lock_mu, init = (int(v) for v in ckt[key + ".residual_meta"].tolist())
                    if not init:
                        res.mu = lock_mu
                        res._after_set_value(p.qparam[0].reshape(-1, 1))      # weight_scale, lock_mu, init = False
                    res.mu, res.init = mu, bool(init)
            else:
                p.data.copy_(ckt[key + ".dense"].to(p.data.device))
            if key + ".opt_step" in ckt:
                st = optimizer.state[p]
                if len(st) == 0:
                    optimizer.init_state(group, p, gi, pi)
                st["step"] = int(ckt[key + ".opt_step"][0])
                for k in _STATE_KEYS:
                    if f"{key}.opt_{k}" in ckt:
                        st[k].copy_(ckt[f"{key}.opt_{k}"].to(st[k].device).view_as(st[k]))
    return int(ckt["meta.step_no"][0])
