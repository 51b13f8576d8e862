"""Host-side mirror of the checkpoint-side modules of `PTQ/quant/quant_linear.py` (the producers and consumers
of the packed-weight layouts on either side of the hot path): `QuantLinearGPTQ`, `QuantLinearA16W4`,
`QuantLinearA8W8`, `matmul248`, `transpose_matmul248`, `quantize_activation_per_token_absmax`.

Same constructor arguments, buffer names / shapes / dtypes (= the `.safetensors` keys) and `pack` / `unpack` /
`forward` semantics as the reference; packing and the GEMMs run on the GPU through liblatentq.  The Triton
kernels of the reference (`matmul_248_kernel`, `transpose_matmul_248_kernel`) are replaced by the tcgen05 dequant
GEMM after an in-memory layout conversion (GPTQ int32 [K/8, N] -> nibble pairs) that is done once per set of
buffers and cached; a general `g_idx` (act-order checkpoints) is served by sorting the input features by group at
conversion time and gathering the activation columns per call.  Tensor-core arithmetic is bf16 here (fp16 in the
reference's Triton kernels), so outputs agree to ~1e-2 relative, not bit for bit.

Citations are `path:line` inside FWkey/latentQ_LLM.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import ops
from .quant import python_compress, python_decompress  # noqa: F401  (same helpers, PTQ/quant/quant_linear.py:400-416)


def _trivial_g_idx(g_idx, infeatures, groupsize):
    want = torch.arange(infeatures, device=g_idx.device, dtype=torch.int64) // groupsize
    return bool(torch.equal(g_idx.to(torch.int64), want))


@torch.no_grad()
def quantize_activation_per_token_absmax(t, n_bits=8):
    """PTQ/quant/quant_linear.py:520-528 (in place, returns the fake-quantized tensor)."""
    assert n_bits == 8
    shape = t.shape
    t2 = t.reshape(-1, shape[-1])
    q, s = ops.act_quant_per_token(t2.to(torch.bfloat16).contiguous())
    t2.copy_((q.float() * s[:, None]).to(t.dtype))
    return t2.view(shape)


def _gptq_as_nibblepair(qweight, scales, qzeros, maxq, N, K, groupsize):
    """GPTQ buffers -> (codes, scales, zeros) in the layout the GEMM consumes.  zero = (stored + 1) & maxq as in
    matmul_248_kernel (PTQ/quant/quant_linear.py:120-121)."""
    codes = ops.gptq_to_nibblepair(qweight.contiguous(), N, K)
    G = K // groupsize
    shifts = torch.arange(0, 32, 4, device=qzeros.device, dtype=torch.int32)
    z = ((qzeros.unsqueeze(-1) >> shifts) & maxq).reshape(G, -1)[:, :N]          # [G, N]
    z = ((z + 1) & maxq).t().contiguous().reshape(-1).to(torch.bfloat16)         # [N*G]
    s = scales.t().contiguous().reshape(-1).to(torch.bfloat16)
    return codes, s, z


# Converted weights per set of GPTQ buffers: the layout conversion (a full pass over the weights) and the inspection of
# g_idx (a host synchronisation) happen once, not per call.  Keyed by the buffers' storage and in-place version counters,
# so `pack`, `load_state_dict` or any in-place edit makes a new entry; bounded.
_GPTQ_CACHE: dict = {}
_GPTQ_CACHE_MAX = 1024


def _gptq_prepared(qweight, scales, qzeros, g_idx, maxq):
    """(codes, scales, zeros, perm, inv_perm, N, K, groupsize) for the GEMM.  `perm` is None for the exporter's
    g_idx = k // groupsize.  A general g_idx (act-order checkpoints: input feature k uses the scale / zero row
    g_idx[k], PTQ/quant/quant_linear.py:113-122) is handled by sorting the input features by group once: the weight rows
    are stored in that order, and a call gathers the activation columns with `perm` (or scatters the grad-input back)."""
    key = tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in (qweight, scales, qzeros, g_idx))
    hit = _GPTQ_CACHE.get(key)
    if hit is not None:
        return hit
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    groupsize = K // scales.shape[0]
    perm = inv_perm = None
    qw = qweight
    if not _trivial_g_idx(g_idx, K, groupsize):
        gi = g_idx.to(torch.int64)
        counts = torch.bincount(gi, minlength=scales.shape[0])
        if counts.numel() != scales.shape[0] or not bool((counts == groupsize).all()):
            raise NotImplementedError("g_idx must assign exactly `groupsize` input features to every group")
        perm = torch.argsort(gi, stable=True)
        inv_perm = torch.empty_like(perm)
        inv_perm[perm] = torch.arange(K, device=perm.device)
        # reorder the weight rows (input features) by group: unpack [K/8, N] words to one code per k, gather, repack
        shifts = torch.arange(0, 32, 4, device=qweight.device, dtype=torch.int32)
        codes_kn = ((qweight.unsqueeze(1) >> shifts.view(1, 8, 1)) & 15).reshape(K, N)
        codes_kn = codes_kn.index_select(0, perm).view(K // 8, 8, N)
        qw = torch.zeros((K // 8, N), dtype=torch.int64, device=qweight.device)
        for j in range(8):
            qw |= codes_kn[:, j, :].to(torch.int64) << (4 * j)
        qw = torch.where(qw >= 2 ** 31, qw - 2 ** 32, qw).to(torch.int32)
    codes, s, z = _gptq_as_nibblepair(qw, scales, qzeros, maxq, N, K, groupsize)
    if len(_GPTQ_CACHE) >= _GPTQ_CACHE_MAX:
        _GPTQ_CACHE.clear()
    out = _GPTQ_CACHE[key] = (codes, s, z, perm, inv_perm, N, K, groupsize)
    return out


def matmul248(input, qweight, scales, qzeros, g_idx, bits, maxq):
    """PTQ/quant/quant_linear.py:263-269: input[M,K] · deq(qweight)[K,N] -> fp16 [M,N]."""
    assert bits == 4
    codes, s, z, perm, _, N, K, groupsize = _gptq_prepared(qweight, scales, qzeros, g_idx, maxq)
    x = input.to(torch.bfloat16)
    x = x.index_select(1, perm) if perm is not None else x.contiguous()
    y = ops.gemm_a16w4_fwd(x, codes, s, z, None, N, K, groupsize)
    return y.to(torch.float16)


def transpose_matmul248(input, qweight, scales, qzeros, g_idx, bits, maxq):
    """PTQ/quant/quant_linear.py:272-279: grad-input, input[M,N] · deq(qweight)^T -> fp16 [M,K]."""
    assert bits == 4
    codes, s, z, _, inv_perm, N, K, groupsize = _gptq_prepared(qweight, scales, qzeros, g_idx, maxq)
    dx = ops.gemm_a16w4_dgrad(input.to(torch.bfloat16).contiguous(), codes, s, z, N, K, groupsize)
    if inv_perm is not None:
        dx = dx.index_select(1, inv_perm)
    return dx.to(torch.float16)


class QuantLinearFunction(torch.autograd.Function):
    """PTQ/quant/quant_linear.py:282-301."""

    @staticmethod
    def forward(ctx, input, qweight, scales, qzeros, g_idx, bits, maxq):
        ctx.save_for_backward(qweight, scales, qzeros, g_idx)
        ctx.bits, ctx.maxq = bits, maxq
        return matmul248(input, qweight, scales, qzeros, g_idx, bits, maxq)

    @staticmethod
    def backward(ctx, grad_output):
        qweight, scales, qzeros, g_idx = ctx.saved_tensors
        grad_input = None
        if ctx.needs_input_grad[0]:
            grad_input = transpose_matmul248(grad_output, qweight, scales, qzeros, g_idx, ctx.bits, ctx.maxq)
        return grad_input, None, None, None, None, None, None


class QuantLinearGPTQ(nn.Module):
    """PTQ/quant/quant_linear.py:304-396."""

    def __init__(self, bits, groupsize, infeatures, outfeatures, bias):
        super().__init__()
        if bits not in [2, 4, 8]:
            raise NotImplementedError("Only 2,4,8 bits are supported.")
        if bits != 4:
            raise NotImplementedError("this build packs 4-bit weights only")
        self.infeatures, self.outfeatures, self.bits = infeatures, outfeatures, bits
        self.maxq = 2 ** bits - 1
        self.groupsize = groupsize if groupsize != -1 else infeatures
        G = math.ceil(infeatures / self.groupsize)
        self.register_buffer('qweight', torch.zeros((infeatures // 32 * bits, outfeatures), dtype=torch.int32))
        self.register_buffer('qzeros', torch.zeros((G, outfeatures // 32 * bits), dtype=torch.int32))
        self.register_buffer('scales', torch.zeros((G, outfeatures), dtype=torch.float16))
        self.register_buffer('g_idx', torch.tensor([i // self.groupsize for i in range(infeatures)], dtype=torch.int32))
        if bias:
            self.register_buffer('bias', torch.zeros((outfeatures), dtype=torch.float16))
        else:
            self.bias = None

    @torch.no_grad()
    def pack(self, linear, scales, zeros, g_idx=None):
        """:343-389.  scales / zeros arrive as [N, G]; same arithmetic as the reference's per-column loop,
        vectorised: round((W + zero*scale) / half(scale))."""
        if g_idx is not None:
            self.g_idx = g_idx.clone()
        dev = self.qweight.device if self.qweight.is_cuda else torch.device("cuda")
        W = linear.weight.data.to(dev).float()
        sc = scales.to(dev).float().t().contiguous()            # [G, N]
        zr = zeros.to(dev).float().t().contiguous()
        scale_zeros = zr * sc
        self.scales = sc.clone().half()
        if linear.bias is not None:
            self.bias = linear.bias.clone().half().to(dev)
        gi = self.g_idx.to(dev).long()
        codes = torch.round((W + scale_zeros[gi].t()) / self.scales[gi].t()).to(torch.int32)      # [N, K]
        self.qweight = ops.nibblepair_to_gptq(ops.pack_nibbles((codes & 15).to(torch.uint8).contiguous().view(-1)),
                                              self.outfeatures, self.infeatures)
        # stored zero = zero - 1, packed LSB-first along N with uint32 wrap-around like the reference's numpy code
        zq = ((zr - 1).to(torch.int64) & 0xFFFFFFFF).view(zr.shape[0], -1, 8)      # [G, N/8, 8]
        packed = torch.zeros(zq.shape[:2], dtype=torch.int64, device=dev)
        for j in range(8):
            packed |= (zq[:, :, j] << (4 * j)) & 0xFFFFFFFF
        self.qzeros = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)

    @torch.no_grad()
    def unpack(self, tensor, scales, zeros, g_idx=None):
        """:327-341: fp32 [N, K] = (code - (stored zero + 1)) * scale (no `& maxq` wrap here, as in the reference)."""
        N, K = self.outfeatures, self.infeatures
        codes = ops.unpack_nibbles(ops.gptq_to_nibblepair(tensor.contiguous(), N, K)).view(N, K).to(torch.int8)
        shifts = torch.arange(0, 32, 4, device=zeros.device, dtype=torch.int32)
        z = ((zeros.unsqueeze(-1) >> shifts) & self.maxq).reshape(zeros.shape[0], -1)[:, :N].to(torch.int8)   # [G, N]
        gi = self.g_idx.to(tensor.device).long()
        return ((codes - z[gi].t() - 1) * scales[gi].t()).float()

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.outfeatures,)
        out = QuantLinearFunction.apply(x.reshape(-1, x.shape[-1]), self.qweight, self.scales, self.qzeros, self.g_idx,
                                        self.bits, self.maxq)
        out = out + self.bias if self.bias is not None else out
        return out.reshape(out_shape)


QuantLinear0 = QuantLinearGPTQ


class QuantLinearA16W4(nn.Module):
    """PTQ/quant/quant_linear.py:421-477: producer of the nibble-pair checkpoints that main0.py loads."""

    def __init__(self, bits, groupsize, infeatures, outfeatures, bias):
        super().__init__()
        if bits not in [2, 4, 8]:
            raise NotImplementedError("Only 2,4,8 bits are supported.")
        self.infeatures, self.outfeatures, self.bits = infeatures, outfeatures, bits
        self.maxq = 2 ** bits - 1
        self.fweight = None
        self.groupsize = groupsize if groupsize != -1 else infeatures
        assert infeatures % 32 == 0
        G = math.ceil(infeatures / self.groupsize) * outfeatures
        self.register_buffer('qweight', torch.zeros((infeatures // 8 * bits * outfeatures), dtype=torch.int32))
        self.register_buffer('zeros', torch.zeros((G, 1), dtype=torch.float16))
        self.register_buffer('scales', torch.zeros((G, 1), dtype=torch.float16))
        if bias:
            self.register_buffer('bias', torch.zeros((outfeatures), dtype=torch.float16))
        else:
            self.bias = None

    @torch.no_grad()
    def unpack(self, tensor, g_idx=None):
        if g_idx is not None:
            raise NotImplementedError
        dev = tensor.device
        fint = python_decompress(tensor).view(-1, self.groupsize).float()
        fweight = (fint - self.zeros.to(dev)) * self.scales.to(dev)
        return fweight.view(self.outfeatures, self.infeatures).half()

    @torch.no_grad()
    def pack(self, linear, scales, zeros, g_idx=None):
        dev = torch.device("cuda")
        self.scales = scales.contiguous().half().reshape(-1, 1).to(dev)
        self.zeros = zeros.contiguous().half().reshape(-1, 1).to(dev)
        self.fweight = linear.weight.data.cpu().clone()
        if linear.bias is not None:
            self.bias = linear.bias.clone().half().to(dev)
        W = linear.weight.data.contiguous().to(dev)
        intweight = torch.round(W.view(-1, self.groupsize).float() / self.scales + self.zeros).to(torch.int)
        self.qweight = python_compress(intweight)

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.outfeatures,)
        s = self.scales.reshape(-1).to(torch.bfloat16)
        z = self.zeros.reshape(-1).to(torch.bfloat16)
        out = ops.gemm_a16w4_fwd(x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous(), self.qweight, s, z, None,
                                 self.outfeatures, self.infeatures, self.groupsize).to(x.dtype)
        out = out + self.bias if self.bias is not None else out
        return out.reshape(out_shape)


QuantLinear2 = QuantLinearA16W4


class QuantLinearA8W8(nn.Module):
    """PTQ/quant/quant_linear.py:578-719 (8-bit weights; the static activation clamp of `forward`)."""

    def __init__(self, bits, groupsize, infeatures, outfeatures, bias):
        super().__init__()
        if bits != 8:
            raise NotImplementedError("this build packs 8-bit weights only")
        assert groupsize == -1
        self.infeatures, self.outfeatures, self.bits = infeatures, outfeatures, bits
        self.maxq = 2 ** bits - 1
        self.name = ''
        self.register_buffer('inp_absmax', torch.zeros((infeatures), dtype=torch.float16))
        self.register_buffer('out_scale', torch.zeros((outfeatures), dtype=torch.float16))
        self.input_bias = None
        self.register_buffer('qweight', torch.zeros((outfeatures, infeatures), dtype=torch.uint8))
        self.register_buffer('qzeros', torch.zeros((outfeatures, 1), dtype=torch.int16))
        self.register_buffer('scales', torch.zeros((outfeatures, 1), dtype=torch.float16))
        if bias:
            self.register_buffer('bias', torch.zeros((outfeatures), dtype=torch.float16))
        else:
            self.bias = None
        self.clampv = None

    def set_clampv(self, up_scale=1.0):
        self.inp_absmax *= up_scale
        self.clampv = self.inp_absmax.max().item()

    @torch.no_grad()
    def unpack(self, tensor):
        return ((tensor - self.qzeros) * self.scales).to(self.scales.dtype)

    @torch.no_grad()
    def pack(self, linear, scales, zeros, g_idx=None):
        """:668-692: qweight = uint8(round((W + zero*scale) / half(scale)))."""
        dev = torch.device("cuda")
        scales = scales.reshape(-1, 1).to(dev).float()
        zeros = zeros.reshape(-1, 1).to(dev).float()
        self.scales = scales.clone().half()
        if linear.bias is not None:
            self.bias = linear.bias.clone().half().to(dev)
        W = linear.weight.data.to(dev).float()
        self.qweight = torch.round((W + zeros * scales) / self.scales).to(torch.uint8)
        self.qzeros = zeros.to(dtype=torch.int16)

    def forward(self, x):
        """:694-719 with the int8 tensor-core GEMM always available (the reference's `except:` fake-quant path and its
        ambiguous `if self.bias:` on a tensor are not reproduced: a bias is used whenever the module has one)."""
        clampv = self.clampv
        if self.input_bias is not None:
            x = x - self.input_bias
        if clampv is not None:
            x = x.clamp(min=-clampv, max=clampv)
        out_shape = x.shape[:-1] + (self.outfeatures,)
        Am = (x * 127. / clampv).round().clamp(-127, 127).view(-1, x.shape[-1]).to(torch.int8).contiguous()
        Bm = (self.qweight.to(torch.int16) - self.qzeros).to(torch.int8).contiguous()
        sc = self.scales.view(-1).to(torch.bfloat16)
        b = (self.bias.to(torch.bfloat16) / sc) if self.bias is not None else 0 * sc
        out = ops.gemm_a8w8(Am, Bm, None, None, clampv / 127., b.contiguous()) * sc.view(1, -1)
        return out.reshape(out_shape).to(x.dtype)


# ---------------------------------------------------------------------------------------------------
# Model surgery and the reference's aliases (PTQ/quant/quant_linear.py:398, 479, 722-770)
# ---------------------------------------------------------------------------------------------------
QuantLinear0 = QuantLinearGPTQ
QuantLinear1 = QuantLinearA8W8
QuantLinear2 = QuantLinearA16W4

config = {'method': 'gptq'}      # 'gptq' -> QuantLinearGPTQ, anything else -> QuantLinearA16W4 (group-wise layers)


def make_quant_linear(module, quantizers, bits, groupsize, name=''):
    """PTQ/quant/quant_linear.py:729-766: replace every sub-module whose qualified name is a key of `quantizers` by an
    (empty) packed layer of the same shape — A8W8 when `groupsize == -1`, otherwise the layout `config['method']`
    selects — carrying over the calibration statistics the PTQ pass attached to the float layer."""
    if isinstance(module, (QuantLinearA8W8, QuantLinearGPTQ, QuantLinearA16W4)):
        return
    for attr, child in list(module.named_children()):
        qualified = f"{name}.{attr}" if name else attr
        if qualified not in quantizers:
            continue
        has_bias = getattr(child, "bias", None) is not None
        if groupsize == -1:
            new = QuantLinearA8W8(bits, groupsize, child.in_features, child.out_features, has_bias)
            if hasattr(child, 'inp_absmax'):
                new.inp_absmax.data = child.inp_absmax
            if hasattr(child, 'inp_bias'):
                new.input_bias = None
                new.register_buffer('input_bias', child.inp_bias)
                new.tmp_bias = torch.nn.functional.linear(child.inp_bias.float(), child.weight.float()).to(torch.float16)
        else:
            cls = QuantLinearGPTQ if config['method'] == 'gptq' else QuantLinearA16W4
            new = cls(bits, groupsize, child.in_features, child.out_features, has_bias)
        new.name = qualified
        if hasattr(new, 'out_scale'):
            if hasattr(child, 'qk_absmax'):
                new.out_scale.data = child.qk_absmax.max()
            if hasattr(child, 'v_absmax'):
                new.out_scale.data = child.v_absmax
        setattr(module, attr, new)
    for attr, child in module.named_children():
        make_quant_linear(child, quantizers, bits, groupsize, f"{name}.{attr}" if name else attr)


def autotune_warmup_linear(model, transpose=False):
    """PTQ/quant/quant_linear.py:772-800 pre-tunes the Triton kernels.  Nothing is tuned here (plans are computed from
    the shape); one call per distinct (K, N) performs the library's one-time per-kernel set-up outside any timed region."""
    seen = set()
    with torch.no_grad():
        for m in model.modules():
            if not isinstance(m, QuantLinearGPTQ) or (m.infeatures, m.outfeatures) in seen:
                continue
            seen.add((m.infeatures, m.outfeatures))
            dev = m.qweight.device
            if dev.type != "cuda":
                continue
            for rows in (1, 64, 2048):
                a = torch.randn(rows, m.infeatures, dtype=torch.float16, device=dev)
                matmul248(a, m.qweight, m.scales, m.qzeros, m.g_idx, m.bits, m.maxq)
                if transpose:
                    a = torch.randn(rows, m.outfeatures, dtype=torch.float16, device=dev)
                    transpose_matmul248(a, m.qweight, m.scales, m.qzeros, m.g_idx, m.bits, m.maxq)
    return len(seen)
