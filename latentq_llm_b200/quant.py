"""Host-side mirror of the reference's `utils/quant.py` for the quantized-weight hot path.

Same names, constructor arguments, attributes, state-dict keys and error behaviour as the reference
module, so that `main0.py:36` / `generate.py:25` (`from utils.quant import MyAdam, QLinearA16W4,
QLinearA8W8, QLinearQAT`) work against this module unchanged.  What differs is below the API: every
quantize / dequantize / pack / GEMM step is one call into liblatentq (hand-written sm_100a kernels)
instead of chains of torch ops, the dequantised weight matrix is never materialised, and there is no
CPU path.

Citations are `path:line` inside FWkey/latentQ_LLM.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Union

import torch
import torch.nn as nn

from . import ops
from .torch_int_shim import linear_a8_w8_bbf16_obf16  # noqa: F401  (re-exported like utils/quant.py:108)

GROUPSIZE = 128  # utils/quant.py:44


def prodx(ls):
    from functools import reduce
    return reduce(lambda x, y: x * y, ls)


# ---------------------------------------------------------------------------------------------------
# functional layer (utils/quant.py:4-103)
# ---------------------------------------------------------------------------------------------------
@torch.no_grad()
def python_compress(fdata, bit=4):
    """utils/quant.py:4-9."""
    assert bit == 4
    return ops.pack_nibbles(fdata.reshape(-1).to(torch.uint8).contiguous())


@torch.no_grad()
def python_decompress(int_data, bit=4):
    """utils/quant.py:12-19; returns int8 [numel/2, 2]."""
    assert bit == 4
    return ops.unpack_nibbles(int_data.contiguous()).view(-1, 2)


@torch.no_grad()
def Qfunc_8bit_opt(tensor, blocksize=1, qparam=None):
    """utils/quant.py:22-33.  `blocksize` is the number of blocks (the reference's naming)."""
    if qparam is not None:
        raise NotImplementedError("quantizing optimizer states with given qparams is not used by the training path")
    shape = tensor.shape
    q, scale, t_max = ops.opt8_quant(tensor.reshape(-1).float().contiguous(), tensor.numel() // blocksize)
    return q.view(shape), [scale, t_max]


@torch.no_grad()
def DeQfunc_8bit_opt(qtensor, qparam, dtype=torch.float32):
    """utils/quant.py:35-41."""
    scale, t_max = qparam
    x = ops.opt8_dequant(qtensor.contiguous(), qtensor.numel() // scale.shape[0], scale.contiguous(), t_max.contiguous())
    return x.view(qtensor.shape).to(dtype)


def _math_dtype(tensor, scales):
    # torch type promotion of `tensor / scales`: bf16 only if both operands are bf16
    return torch.bfloat16 if (tensor.dtype == torch.bfloat16 and scales.dtype == torch.bfloat16) else torch.float32


@torch.no_grad()
def Qfunc_4bit_g_res(tensor, residual_handle, qparam, groupsize=GROUPSIZE):
    """utils/quant.py:45-63 as one fused kernel: Z = w/scale+zero, round, residual encode, carry, clamp, pack."""
    scales, zeros, shape = qparam
    scales = scales.contiguous().reshape(-1)
    zeros = zeros.contiguous().reshape(-1)
    w = tensor.data.contiguous()
    md = _math_dtype(w, scales)
    if isinstance(residual_handle, ResidualTensor):
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=md, res_round_bf16=True,
                          mu_enc=residual_handle.mu)
        qweight, _ = ops.a16w4_requant(w, scales, zeros, o, group=groupsize, words_out=residual_handle.residual_int.view(-1))
        residual_handle._after_set_value(scales.view(-1, 1))
    else:
        residual_handle.data = tensor.view(shape).to(residual_handle.dtype)
        o = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=md)
        qweight, _ = ops.a16w4_requant(w, scales, zeros, o, group=groupsize)
    return qweight


@torch.no_grad()
def DeQfunc_4bit_g(qtensor, qparam, dtype=torch.float32):
    """utils/quant.py:66-72."""
    scales, zeros, shape = qparam
    return ops.a16w4_dequant(qtensor.contiguous(), scales.contiguous().reshape(-1), zeros.contiguous().reshape(-1),
                             tuple(shape), dtype, GROUPSIZE)


@torch.no_grad()
def Qfunc_8bit_res(tensor, residual_handle, qscales):
    """utils/quant.py:88-103 as one fused kernel."""
    w = tensor.contiguous()
    qs = qscales.contiguous().reshape(-1)
    md = _math_dtype(w, qs)
    if residual_handle is None:
        o = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=md)
        q, _ = ops.a8w8_requant(w, qs, o)
    elif isinstance(residual_handle, ResidualTensor):
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=md, res_round_bf16=True,
                          mu_enc=residual_handle.mu)
        q, _ = ops.a8w8_requant(w, qs, o, words_out=residual_handle.residual_int.view(-1))
        residual_handle._after_set_value(qscales)
    else:
        residual_handle.data = tensor.to(residual_handle.dtype)
        o = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=md)
        q, _ = ops.a8w8_requant(w, qs, o)
    return q


# ---------------------------------------------------------------------------------------------------
# autograd functions (utils/quant.py:109-394)
# ---------------------------------------------------------------------------------------------------
dict_temp = []  # utils/quant.py:109-110: weight gradients travel from backward() to the module hook through this list


def _w4_args(qparamw4):
    scales, zeros, shape = qparamw4
    return scales.contiguous().reshape(-1), zeros.contiguous().reshape(-1), int(shape[0]), int(shape[1])


class QLinearFunctionW4(torch.autograd.Function):
    """utils/quant.py:112-146.  forward: x·deq(W)^T (+bias); backward: dY·deq(W), dY^T·x (dense, to `dict_temp`)."""

    @staticmethod
    def forward(input, weight_d, qparamw4, bias):
        s, z, N, K = _w4_args(qparamw4)
        return ops.gemm_a16w4_fwd(input.contiguous(), weight_d, s, z, None if bias is None else bias.data.contiguous(), N, K,
                                  GROUPSIZE)

    @staticmethod
    def setup_context(ctx, inputs, output):
        input, weight_d, qparamw4, bias = inputs
        ctx.save_for_backward(input, weight_d.data, bias)
        ctx.save_qparamw4 = qparamw4

    @staticmethod
    def backward(ctx, grad_output):
        input, weight_d, bias = ctx.saved_tensors
        s, z, N, K = _w4_args(ctx.save_qparamw4)
        grad_output = grad_output.contiguous()
        grad_input = grad_bias = None
        if ctx.needs_input_grad[0]:
            grad_input = ops.gemm_a16w4_dgrad(grad_output, weight_d, s, z, N, K, GROUPSIZE)
        grad_weight = grad_output.t().mm(input)
        dict_temp.append(grad_weight)
        # The reference tests needs_input_grad[2] here (:143) — the slot of the qparam list, never True — so the
        # bias of a quantized linear receives no gradient.  Reproduced: it decides which parameters get trained.
        if bias is not None and ctx.needs_input_grad[2]:
            grad_bias = grad_output.sum(0)
        return grad_input, None, None, grad_bias


# The hook-free route's weight gradient dY^T·X is a plain dense bf16 GEMM with beta = 1.  Default: the library GEMM
# (`addmm_`).  LQ_WGRAD_TCGEN05=1 (read at import) selects this package's tcgen05 kernel `ops.gemm_wgrad` instead: same
# single rounding of the fp32 sum, measured at 0.65-0.85 of the library's rate on the fine-tune shapes (one-CTA 128 x 256
# tiles keep the shared-memory port busy with 12 KB of operand reads per MMA on top of the TMA writes; the library pairs
# CTAs on 256 x 256 tiles).
_WGRAD_TCGEN05 = bool(os.environ.get("LQ_WGRAD_TCGEN05"))


class QLinearFunctionW4Direct(torch.autograd.Function):
    """Hook-free variant of QLinearFunctionW4 for this package's own trainer: same forward and grad-input, but the
    weight gradient dY^T·x is accumulated straight into `qtensor.grad` (a view of the data-parallel gradient arena)
    by one GEMM with beta = 1 (the library's, or `ops.gemm_wgrad`: tcgen05, both operands MN-major straight from their
    row-major tensors; both round the fp32 sum once into the arena) instead of travelling through `dict_temp` and a module
    backward hook (utils/quant.py:141-142, 398-411).  No [N, K] temporary, no extra add pass, no hook overhead."""

    @staticmethod
    def forward(ctx, input, weight_d, scales, zeros, bias, qtensor, N, K):
        ctx.save_for_backward(input, weight_d, scales, zeros)
        ctx.qtensor, ctx.N, ctx.K = qtensor, N, K
        return ops.gemm_a16w4_fwd(input, weight_d, scales, zeros, None if bias is None else bias.data, N, K, GROUPSIZE)

    @staticmethod
    def backward(ctx, grad_output):
        input, weight_d, scales, zeros = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        grad_input = None
        if ctx.needs_input_grad[0]:
            grad_input = ops.gemm_a16w4_dgrad(grad_output, weight_d, scales, zeros, ctx.N, ctx.K, GROUPSIZE)
        q = ctx.qtensor
        x2 = input if input.is_contiguous() else input.contiguous()
        if not _WGRAD_TCGEN05 or ctx.N % 8 or ctx.K % 8:
            if q.grad is None:
                q.grad = grad_output.t().mm(x2)
            else:
                q.grad.addmm_(grad_output.t(), x2)
        elif q.grad is None:
            q.grad = ops.gemm_wgrad(grad_output, x2)
        else:
            ops.gemm_wgrad(grad_output, x2, q.grad, accumulate=True)
        return grad_input, None, None, None, None, None, None, None


class QLinearFunctionW4_eval(torch.autograd.Function):
    """utils/quant.py:149-169."""

    @staticmethod
    def forward(input, weight_d, qparamw4, bias):
        s, z, N, K = _w4_args(qparamw4)
        return ops.gemm_a16w4_fwd(input.contiguous(), weight_d, s, z, None if bias is None else bias.data.contiguous(), N, K,
                                  GROUPSIZE)

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, grad_output):
        return None, None, None, None


def _a8w8_forward(input8, clampv, weight_d, qscales, bias):
    """The reference's call `linear_a8_w8_bbf16_obf16(x8, w8, bias/qscales, clampv/127.) * qscales`
    (utils/quant.py:268-271).  `clampv` is a Python float (static) or a device tensor (dynamic: input.max());
    the tensor case avoids the host synchronisation of converting it to a float."""
    M = input8.shape[0]
    if torch.is_tensor(clampv):
        # clampv/127. on the reference's 0-dim bf16 tensor rounds to bf16
        alpha = (clampv.to(torch.bfloat16) / 127.).float().reshape(1).expand(M).contiguous()
    else:
        alpha = torch.full((M,), float(clampv) / 127., dtype=torch.float32, device=input8.device)
    if bias is not None:
        b = (bias / qscales.view(-1)).to(torch.bfloat16).contiguous()
    else:
        b = (0 * qscales.view(-1)).to(torch.bfloat16).contiguous()
    out = ops.gemm_a8w8(input8, weight_d, alpha, None, 1.0, b)
    return out * qscales.view(1, -1)


def _quant_input_static(input, clampv):
    """input*127./clampv ; round ; clamp(-128,127) -> int8 (utils/quant.py:178-179) with a given clampv."""
    input8 = input * 127. / clampv
    return input8.round_().clamp_(-128, 127).to(torch.int8)


def _a8w8_backward(ctx, grad_output, input_f, weight_d, qscales, bias, detach=False):
    weight_forward = weight_d.to(grad_output.dtype) * qscales
    grad_input = grad_bias = None
    if ctx.needs_input_grad[0]:
        grad_input = grad_output.mm(weight_forward)
    grad_weight = grad_output.t().mm(input_f)
    dict_temp.append(grad_weight.data if detach else grad_weight)
    if bias is not None and ctx.needs_input_grad[2]:     # same slot as the reference (:208, :249, :290)
        grad_bias = grad_output.sum(0)
    return grad_input, None, None, grad_bias


class QLinearFunctionA8W8_static(torch.autograd.Function):
    """utils/quant.py:172-211."""

    @staticmethod
    def forward(input, weight_d, qparamaw, bias):
        clampv, qscales = qparamaw
        return _a8w8_forward(_quant_input_static(input, clampv), float(clampv), weight_d, qscales, bias)

    @staticmethod
    def setup_context(ctx, inputs, output):
        input, weight_d, qparamaw, bias = inputs
        ctx.save_for_backward(input, weight_d.data, bias)
        ctx.save_qparamaw = qparamaw

    @staticmethod
    def backward(ctx, grad_output):
        input, weight_d, bias = ctx.saved_tensors
        clampv, qscales = ctx.save_qparamaw
        int_s = 127. / clampv
        input_f = (input * int_s).round_().clamp_(-128, 127).div_(int_s)
        return _a8w8_backward(ctx, grad_output, input_f, weight_d, qscales, bias)


class QLinearFunctionA8W8_dynamic(torch.autograd.Function):
    """utils/quant.py:254-293.  Forward as written; backward uses the working arithmetic of
    `QLinearFunctionA8W8_dynamic0.backward` (:235-252) — the in-place `weight_d *= qscales` on an int8
    tensor at :281-283 raises in torch and is not reproduced."""

    @staticmethod
    def forward(ctx, input, weight_d, qparamaw, bias):
        _, qscales = qparamaw
        input8, clampv = ops.act_quant_per_tensor(input.contiguous())      # clampv = input.max() on device (:260)
        ctx.save_qparamaw = (clampv, qscales)
        ctx.save_for_backward(input8, weight_d.data, bias)
        return _a8w8_forward(input8, clampv, weight_d, qscales, bias)

    @staticmethod
    def backward(ctx, grad_output):
        input8, weight_d, bias = ctx.saved_tensors
        clampv, qscales = ctx.save_qparamaw
        int_s = (clampv.to(grad_output.dtype) / 127.)
        input_f = input8.to(grad_output.dtype) * int_s
        return _a8w8_backward(ctx, grad_output, input_f, weight_d, qscales, bias, detach=True)


QLinearFunctionA8W8_dynamic0 = QLinearFunctionA8W8_dynamic   # utils/quant.py:214-252 (same arithmetic, host-synchronising)


class QLinearFunctionA8W8_static_eval(torch.autograd.Function):
    """utils/quant.py:296-312."""

    @staticmethod
    def forward(ctx, input, weight_d, qparamaw, bias):
        clampv, qscales = qparamaw
        return _a8w8_forward(_quant_input_static(input, clampv), float(clampv), weight_d, qscales, bias)

    @staticmethod
    def backward(ctx, grad_output):
        return None, None, None, None


class QLinearFunctionA8W8_dynamic_eval(torch.autograd.Function):
    """utils/quant.py:314-331."""

    @staticmethod
    def forward(ctx, input, weight_d, qparamaw, bias):
        _, qscales = qparamaw
        input8, clampv = ops.act_quant_per_tensor(input.contiguous())
        return _a8w8_forward(input8, clampv, weight_d, qscales, bias)

    @staticmethod
    def backward(ctx, grad_output):
        return None, None, None, None


def _qat_weight(weight_f, qscales):
    q, _ = ops.a8w8_requant(weight_f.contiguous(), qscales.contiguous().reshape(-1),
                            ops.make_opts(codec=ops.CODEC_NONE, math_dtype=_math_dtype(weight_f, qscales)))
    return q


class QLinearFunctionQAT_dynamic(torch.autograd.Function):
    """utils/quant.py:334-374."""

    @staticmethod
    def forward(ctx, input, weight_f, qparamaw, bias):
        _, qscales = qparamaw
        input8, clampv = ops.act_quant_per_tensor(input.contiguous())
        ctx.save_for_backward(input, weight_f.data, bias)
        ctx.save_qparamaw = (clampv, qscales)
        return _a8w8_forward(input8, clampv, _qat_weight(weight_f, qscales), qscales, bias)

    @staticmethod
    def backward(ctx, grad_output):
        input, weight_f, bias = ctx.saved_tensors
        clampv, qscales = ctx.save_qparamaw
        int_s = 127. / clampv.to(input.dtype)
        input_f = (input * int_s).round_().clamp_(-128, 127).div_(int_s)
        weight_d = _qat_weight(weight_f, qscales)
        return _a8w8_backward(ctx, grad_output, input_f, weight_d, qscales, bias)


class QLinearFunctionQAT_dynamic_eval(torch.autograd.Function):
    """utils/quant.py:376-394."""

    @staticmethod
    def forward(ctx, input, weight_f, qparamaw, bias):
        _, qscales = qparamaw
        input8, clampv = ops.act_quant_per_tensor(input.contiguous())
        return _a8w8_forward(input8, clampv, _qat_weight(weight_f, qscales), qscales, bias)

    @staticmethod
    def backward(ctx, grad_output):
        return None, None, None, None


def backward_hook_fn(module, grad_out, grad_in):
    """utils/quant.py:398-411."""
    assert len(dict_temp) == 1
    if isinstance(module.weight.grad, GradientQTensor):
        if module.weight.grad.acc_ite == 0:
            module.weight.grad.set_value(dict_temp.pop())
        else:
            module.weight.grad.add_(dict_temp.pop())
    else:
        if module.weight.grad is None:
            module.weight.grad = dict_temp.pop()
        else:
            module.weight.grad.add_(dict_temp.pop())


# ---------------------------------------------------------------------------------------------------
# modules (utils/quant.py:413-599)
# ---------------------------------------------------------------------------------------------------
class QLinearA16W4(nn.Module):
    """utils/quant.py:413-482."""

    def __init__(self, input_features, output_features, bias=True, lbit=0, gbit=16):
        super().__init__()
        self.input_features = input_features
        self.output_features = output_features
        if bias:
            self.bias = nn.Parameter(torch.empty(output_features))
        else:
            self.register_parameter('bias', None)
        self.groupsize = groupsize = GROUPSIZE
        n_groups = math.ceil(input_features / groupsize) * output_features
        self.register_buffer('qweight', torch.tensor([]))
        self.register_buffer('zeros', torch.zeros((n_groups, 1), dtype=torch.bfloat16))
        self.register_buffer('scales', torch.zeros((n_groups, 1), dtype=torch.bfloat16))
        self.weight = QuantTensor([output_features, input_features], lbit=lbit, wbit=4, gbit=gbit)
        self.wshape = [output_features, input_features]
        self.hook_handle = None

    def add_hook(self, direct=False):
        """`direct=False`: the reference's full backward hook (utils/quant.py:435-436).  `direct=True` (an extension
        used by this package's trainer): no hook, the weight gradient is accumulated into `weight.grad` by the
        autograd function itself."""
        if direct:
            self.hook_handle = "direct"
            self._flat_qparams = None
        else:
            self.hook_handle = self.register_full_backward_hook(backward_hook_fn)

    def before_save(self):
        self.qweight.data = self.weight.data.cpu()

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.output_features,)
        if self.hook_handle == "direct":
            fq = self._flat_qparams
            if fq is None or fq[2] is not self.weight.qparam:
                sc, zr, _ = self.weight.qparam
                fq = self._flat_qparams = (sc.contiguous().reshape(-1), zr.contiguous().reshape(-1), self.weight.qparam)
            x2 = x.reshape(-1, x.shape[-1])
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            out = QLinearFunctionW4Direct.apply(x2, self.weight.data, fq[0], fq[1], self.bias, self.weight,
                                                self.output_features, self.input_features)
            return out.reshape(out_shape)
        fn = QLinearFunctionW4_eval if self.hook_handle is None else QLinearFunctionW4
        out = fn.apply(x.reshape(-1, x.shape[-1]), self.weight.data, self.weight.qparam, self.bias)
        return out.reshape(out_shape)

    def forward_eval(self, x):
        out_shape = x.shape[:-1] + (self.output_features,)
        out = QLinearFunctionW4_eval.apply(x.reshape(-1, x.shape[-1]), self.weight.data, self.weight.qparam, self.bias)
        return out.reshape(out_shape)

    def to(self, device: Optional[Union[int, torch.device]]):
        self.weight = self.weight.to(device=device)
        self.zeros = self.zeros.to(device=device)
        self.scales = self.scales.to(device=device)
        self.weight.set_value(None, [self.scales, self.zeros, self.wshape])
        if self.bias is not None:
            self.bias.data = self.bias.data.to(device)

    def extra_repr(self):
        return 'QLinearA16W4 input_features={}, output_features={}, bias={}'.format(
            self.input_features, self.output_features, self.bias is not None)


class QLinearA8W8(nn.Module):
    """utils/quant.py:485-541."""

    def __init__(self, input_features, output_features, bias=True, lbit=0, gbit=8):
        super().__init__()
        self.input_features = input_features
        self.output_features = output_features
        if bias:
            self.bias = nn.Parameter(torch.empty(output_features))
        else:
            self.register_parameter('bias', None)
        self.register_buffer('qweight', torch.tensor([]))
        self.register_buffer('clampv', torch.ones(1))
        self.register_buffer('qscales', torch.zeros(output_features, 1, dtype=torch.bfloat16))
        self.weight = QuantTensor([output_features, input_features], lbit=lbit, wbit=8, gbit=gbit)
        self.wshape = [output_features, input_features]
        self.hook_handle = None

    def add_hook(self):
        self.hook_handle = self.register_full_backward_hook(backward_hook_fn)

    def before_save(self):
        self.qweight.data = self.weight.data.cpu()

    def _qparam(self):
        # the reference passes clampv.item(); the dynamic functions ignore it and take input.max()
        return (self.clampv, self.qscales.data)

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.output_features,)
        fn = QLinearFunctionA8W8_dynamic_eval if self.hook_handle is None else QLinearFunctionA8W8_dynamic
        out = fn.apply(x.reshape(-1, x.shape[-1]), self.weight.data, self._qparam(), self.bias)
        return out.reshape(out_shape)

    def forward_eval(self, x):
        out_shape = x.shape[:-1] + (self.output_features,)
        out = QLinearFunctionA8W8_dynamic_eval.apply(x.reshape(-1, x.shape[-1]), self.weight.data, self._qparam(), self.bias)
        return out.reshape(out_shape)

    def to(self, device: Optional[Union[int, torch.device]]):
        self.weight = self.weight.to(device=device)
        self.qscales = self.qscales.to(device=device)
        self.weight.set_value(None, self.qscales)
        if self.bias is not None:
            self.bias.data = self.bias.data.to(device)

    def extra_repr(self):
        return 'QLinearA8W8 input_features={}, output_features={}, bias={}'.format(
            self.input_features, self.output_features, self.bias is not None)


class QLinearQAT(nn.Module):
    """utils/quant.py:544-599."""

    def __init__(self, input_features, output_features, bias=True, lbit=0, gbit=16):
        super().__init__()
        self.input_features = input_features
        self.output_features = output_features
        if bias:
            self.bias = nn.Parameter(torch.empty(output_features))
        else:
            self.register_parameter('bias', None)
        self.register_buffer('qweight', torch.tensor([]))
        self.register_buffer('clampv', torch.ones(1))
        self.register_buffer('qscales', torch.zeros(output_features, 1, dtype=torch.bfloat16))
        assert gbit == 16
        self.weight = FPTensor(torch.empty((output_features, input_features), dtype=torch.bfloat16))
        self.wshape = [output_features, input_features]
        self.hook_handle = None

    def add_hook(self):
        self.hook_handle = self.register_full_backward_hook(backward_hook_fn)

    def before_save(self):
        self.qweight.data = _qat_weight(self.weight.data, self.qscales).cpu()

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.output_features,)
        fn = QLinearFunctionQAT_dynamic_eval if self.hook_handle is None else QLinearFunctionQAT_dynamic
        out = fn.apply(x.reshape(-1, x.shape[-1]), self.weight.data, (self.clampv, self.qscales.data), self.bias)
        return out.reshape(out_shape)

    def forward_eval(self, x):
        out_shape = x.shape[:-1] + (self.output_features,)
        out = QLinearFunctionQAT_dynamic_eval.apply(x.reshape(-1, x.shape[-1]), self.weight.data,
                                                    (self.clampv, self.qscales.data), self.bias)
        return out.reshape(out_shape)

    def to(self, device: Optional[Union[int, torch.device]]):
        self.weight = self.weight.to(device=device)
        if self.bias is not None:
            self.bias.data = self.bias.data.to(device)

    def extra_repr(self):
        return 'QLinearQAT input_features={}, output_features={}, bias={}'.format(
            self.input_features, self.output_features, self.bias is not None)


# ---------------------------------------------------------------------------------------------------
# parameter containers (utils/quant.py:606-705, 790-921)
# ---------------------------------------------------------------------------------------------------
class QuantTensor(object):
    """utils/quant.py:606-663."""

    def __init__(self, shape, wbit=8, gbit=8, lbit=4):
        self.shape = shape
        self.wbit = wbit
        self.initial = False
        self.qparam = None
        self.lbit = lbit
        if lbit == 4:
            num_channels = shape[0] if wbit == 8 else prodx(self.shape) // GROUPSIZE
            qshape = [num_channels, prodx(self.shape) // num_channels]
            self.residual = ResidualTensor(qshape=qshape, oshape=shape)
        else:
            self.residual = torch.empty(shape, dtype=torch.bfloat16 if lbit == 16 else torch.float32)
        self.requires_grad = True
        self.grad = None if gbit == 16 else GradientQTensor(self.shape, bit=gbit)

    def set_value(self, data, qparam=None):
        if data is not None:
            self.data = data.clone()
        self.qparam = qparam
        self.initial = True
        self.requires_grad = True

    def numel(self):
        return prodx(self.shape)

    def get_self(self):
        return self

    def __repr__(self):
        return "Quant value:\n{}\n with param:\n{}".format(self.data, self.qparam)

    def requires_grad_(self, boolv):
        self.requires_grad = boolv
        return self

    def to(self, device=None, dtype=None):
        if device is not None:
            self.data = self.data.to(device)
            if self.lbit > 8:
                self.residual = self.residual.to(device)
        return self

    @property
    def device(self):
        return self.data.device

    @property
    def type(self):
        return self.data.type


class FPTensor(object):
    """utils/quant.py:666-705."""

    def __init__(self, data, gbit=16):
        self.data = data
        self.shape = data.shape
        self.initial = False
        self.qparam = None
        self.requires_grad = True
        self.grad = None if gbit == 16 else GradientQTensor(self.shape, bit=gbit)

    def numel(self):
        return prodx(self.shape)

    def get_self(self):
        return self

    def __repr__(self):
        return "Quant value:\n{}\n with param:\n{}".format(self.data, self.qparam)

    def requires_grad_(self, boolv):
        self.requires_grad = boolv
        return self

    def to(self, device=None, dtype=None):
        if device is not None:
            self.data = self.data.to(device)
        return self

    @property
    def device(self):
        return self.data.device

    @property
    def type(self):
        return self.data.type


def three_fold_curve_4bit(mu):
    """utils/quant.py:708-716."""
    if mu == 3:
        return 2, 0.4330623539159437, 4, 0.46875
    elif mu == 2:
        return 2, 0.37272211741724515, 4, 0.4375
    elif mu == 1:
        return 2, 0.2666300266320331, 4, 0.375
    else:
        return 2, 0.125, 4, 0.25


class _CudaModule:
    """The five functions of the reference's pybind module `MyQuantDequant`
    (utils/cuda_src/multi_random_quant.cpp:38-54), same names and in-place semantics."""

    @staticmethod
    def quant(fp_input, int_input, k1, b1, k2, b2, k3):
        ops.res3_quant(fp_input, int_input, k1, b1, k2, b2, k3, 0.0)

    @staticmethod
    def dequant(int_input, fp_output, k1, b1, k2, b2, k3):
        ops.res3_dequant(int_input, fp_output, k1, b1, k2, b2, k3)

    @staticmethod
    def uniform_quant(fp_input, int_input):
        ops.resu_quant(fp_input, int_input, 0.0)

    @staticmethod
    def uniform_quant_s(fp_input, int_input):
        ops.resu_quant_s(fp_input, int_input)

    @staticmethod
    def uniform_dequant(int_input, fp_output):
        ops.resu_dequant(int_input, fp_output)


cuda_module = _CudaModule()   # utils/quant.py:719
EXT_type = torch.bfloat16     # utils/quant.py:722


@torch.no_grad()
def cuda_quant_linear(residual_fp, q_tensor):
    """utils/quant.py:723-733 (CUDA tensors only: the CPU codec lives in the test oracle, not here)."""
    residual_fp = residual_fp.to(EXT_type)
    assert residual_fp.is_cuda and residual_fp.is_contiguous()
    cuda_module.uniform_quant(residual_fp, q_tensor)
    return residual_fp


@torch.no_grad()
def cuda_quant_3fold(residual_fp, q_tensor, p1, y1, p2, y2):
    """utils/quant.py:735-742."""
    residual_fp = residual_fp.to(EXT_type)
    assert residual_fp.is_cuda and residual_fp.is_contiguous()
    cuda_module.quant(residual_fp, q_tensor, p1, y1, p2 - p1, y2, 8 - p2)
    return residual_fp


@torch.no_grad()
def cuda_dequant_linear(residual_int):
    """utils/quant.py:746-755."""
    assert residual_int.is_cuda and residual_int.is_contiguous()
    fp_tensor = torch.empty((residual_int.numel(), 8), device=residual_int.device, dtype=EXT_type)
    cuda_module.uniform_dequant(residual_int, fp_tensor)
    return fp_tensor


@torch.no_grad()
def cuda_dequant_3fold(residual_int, p1, y1, p2, y2):
    """utils/quant.py:757-763."""
    assert residual_int.is_cuda and residual_int.is_contiguous()
    fp_tensor = torch.empty((residual_int.numel(), 8), device=residual_int.device, dtype=EXT_type)
    cuda_module.dequant(residual_int, fp_tensor, p1, y1, p2 - p1, y2, 8 - p2)
    return fp_tensor


class ResidualTensor(object):
    """utils/quant.py:790-841."""

    def __init__(self, qshape, oshape):
        self.weight_scale = None
        self.qshape = qshape
        self.oshape = oshape
        self.lock_mu = self.mu = 0
        numel_h = prodx(oshape)
        assert numel_h % 8 == 0  # "residual shape must be multiple of 8"
        self.residual_int = torch.empty((numel_h // 8, 1), dtype=torch.int32, device='cuda')
        self.name = 'residual'
        self.init = True

    def _after_set_value(self, weight_scale):
        if weight_scale is not None:
            self.weight_scale = weight_scale
        self.lock_mu = self.mu
        self.init = False

    def set_value(self, residual_fp, weight_scale=None):
        p1, y1, p2, y2 = three_fold_curve_4bit(self.mu)
        adj = cuda_quant_3fold(residual_fp.contiguous(), self.residual_int, p1, y1, p2, y2)
        self._after_set_value(weight_scale)
        return adj

    def update_mu(self, optmizer_std):
        mu = (self.weight_scale / (optmizer_std + 1e-8)).mean().item()
        if mu > 75.8:
            self.mu = 3
        if mu > 36.5:       # as in the reference (:815-818): this second test overrides level 3
            self.mu = 2
        elif mu > 16.2:
            self.mu = 1
        else:
            self.mu = 0
        if self.mu != self.lock_mu:
            print(f'{self.name} now mu level is {mu}({self.mu}), pre is {self.lock_mu}')

    def dequant(self):
        p1, y1, p2, y2 = three_fold_curve_4bit(self.lock_mu)
        return cuda_dequant_3fold(self.residual_int, p1, y1, p2, y2)

    def add(self, tensor: torch.Tensor):
        Tdtype = tensor.dtype
        if not self.init:
            ret = (self.dequant().view(self.qshape) * self.weight_scale).to(dtype=Tdtype).view(self.oshape).add(tensor)
        else:
            ret = tensor
        return ret

    def __repr__(self):
        return "ResidualTensor !"


class GradientQTensor(object):
    """The optional 8-bit stochastic gradient accumulator (utils/quant.py:846-921): one scale per weight row fixed by
    the first micro-batch (4 x its absmax / 127), every later micro-batch folded in as
    `round((q * scale + g) / scale + noise)`.  Same interface as the reference's class; the arithmetic runs in one
    kernel per call (`ops.gradq_accumulate`) with the library's counter-based Philox stream as the noise, keyed by
    (`seed`, call counter), so replicas that feed the same gradients hold the same accumulator."""

    def __init__(self, shape, bit=8, seed=0):
        self.acc_ite = 0
        self.bit = bit
        self.qdata = None
        self.scale = None
        self.qzero = None
        self.shape = shape
        self.fixscale = False
        self.seed = seed
        self.calls = 0

    def _opts(self):
        self.calls += 1
        return ops.make_opts(dither=ops.DITHER_PHILOX, seed=self.seed, step=self.calls, param_id=0x67726164)

    def _kernel(self, fdata, first):
        f2 = fdata.reshape(fdata.shape[0], -1)
        if not f2.is_contiguous():
            f2 = f2.contiguous()
        if first or self.qdata is None or self.qdata.shape != f2.shape or self.scale.dtype != f2.dtype:
            self.qdata = torch.empty(f2.shape, dtype=torch.int8, device=f2.device)
            self.scale = torch.empty(f2.shape[0], dtype=f2.dtype, device=f2.device)
        ops.gradq_accumulate(f2, self.qdata, self.scale, first, self._opts())

    def set_value(self, fdata):
        if self.bit > 8:
            self.qdata = fdata
            return
        self._kernel(fdata, True)
        self.fdtype = fdata.dtype
        self.acc_ite = 1

    def zero(self):
        self.acc_ite = 0
        if self.bit > 8:
            self.qdata = None

    def add_(self, fdata):
        if self.bit > 8:
            self.qdata += fdata
        else:
            self.acc_ite += 1
            self._kernel(fdata, False)

    def dequant(self):
        return ops.gradq_dequant(self.qdata, self.scale).view(*self.shape)

    def get_value(self):
        return self.qdata if self.bit > 8 else self.dequant()

    def __repr__(self):
        return f"GradientQTensor bitwidth {self.bit} !"

    def to(self, device):
        if self.qdata is not None:
            self.qdata = self.qdata.to(device)
        if self.bit <= 8 and self.scale is not None:
            self.scale = self.scale.to(device)
        return self

    @property
    def device(self):
        return self.qdata.device


# ---------------------------------------------------------------------------------------------------
# optimizer (utils/quant.py:927-1148)
# ---------------------------------------------------------------------------------------------------
class MyAdam(torch.optim.Adam):
    """utils/quant.py:927-1148.  Same constructor and state layout (`state1/state2` uint8, `qmap*` = scale,
    `absmax*` = t_max per block of 2048 / 128 elements, second state holds sqrt(v)+eps).  The per-parameter
    device synchronisation and allocator flush of the reference (:985, :1137) are not reproduced.

    `fused=True` (default, an extension): a quantized A16W4 weight with 8-bit states takes ONE kernel per step
    (`ops.adam_a16w4_step`: same arithmetic, every intermediate rounded where the tensor ops below round it, so
    codes / residual / states are bit-identical to the op-by-op route), and all small dense bf16 parameters of a
    group take one launch together.  Steps that also refresh the residual-curve level (:1107-1111), parameters
    with weight decay, CPU-resident states and every other layout use `update_step`, the op-by-op route."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), obit=8, mu_updata_f=20, cpu=False, fused=True):
        super().__init__(params, lr=lr, betas=betas)
        self.initialized = False
        self.obit = obit
        self.mu_updata_f = mu_updata_f
        self.statedevice = 'cpu' if cpu else 'cuda'
        self.fused = bool(fused) and not cpu
        self.before_param = None                 # optional callable(p), run before a parameter with a gradient is stepped
        self.last_to_first = False               # walk each group's parameters from the last to the first (see step)
        self.op_by_op_steps = 0                  # parameter steps that took `update_step` instead of a fused kernel
        self._dense_tables = {}

    def add_param_group(self, param_group):
        assert isinstance(param_group, dict), "param group must be a dict"
        params = param_group['params']
        if isinstance(params, torch.Tensor):
            param_group['params'] = [params]
        elif isinstance(params, set):
            raise TypeError('optimizer parameters need to be organized in ordered collections, but '
                            'the ordering of tensors in sets will change between runs. Please use a list instead.')
        else:
            param_group['params'] = list(params)
        for name, default in self.defaults.items():
            param_group.setdefault(name, default)
        param_set = set()
        for group in self.param_groups:
            param_set.update(set(group['params']))
        if not param_set.isdisjoint(set(param_group['params'])):
            raise ValueError("some parameters appear in more than one parameter group")
        self.param_groups.append(param_group)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        dense = {}
        for gindex, group in enumerate(self.param_groups):
            # Parameters are independent of one another (dither streams are keyed by parameter, not by visiting order),
            # so the walk may run backwards: a data-parallel step then meets the gradients in the order their
            # all-reduces were queued during the backward pass (last layers first) instead of waiting for the whole
            # queue before the first parameter.
            walk = list(enumerate(group["params"]))
            for pindex, p in (reversed(walk) if self.last_to_first else walk):
                if p.grad is None:
                    continue
                if self.before_param is not None:           # data-parallel step: wait for this gradient's all-reduce only
                    self.before_param(p)
                state = self.state[p]
                if len(state) == 0:
                    self.init_state(group, p, gindex, pindex)
                if self.fused and self._fused_quant_ok(group, p, state):
                    self._fused_quant_step(group, p, state)
                elif self.fused and self._fused_dense_ok(group, p, state):
                    dense.setdefault((gindex, state["step"]), []).append(p)
                else:
                    self.op_by_op_steps += 1
                    self.update_step(group, p, gindex, pindex)
        for (gindex, _), plist in dense.items():
            self._fused_dense_step(gindex, self.param_groups[gindex], plist)
        return loss

    # ---- fused routes -----------------------------------------------------------------------------
    def _step_size(self, group, step):
        beta1, beta2 = group["betas"]
        return group["lr"] * math.sqrt(1 - beta2 ** step) / (1 - beta1 ** step)

    def _fused_quant_ok(self, group, p, state):
        if not (isinstance(p, QuantTensor) and p.wbit in (4, 8) and isinstance(p.residual, ResidualTensor)):
            return False
        g = p.grad
        if isinstance(g, GradientQTensor):
            return g.bit <= 8 and g.qdata is not None and g.qdata.is_cuda
        if not (torch.is_tensor(g) and g.is_cuda and g.is_contiguous() and g.dtype in (torch.bfloat16, torch.float32)):
            return False
        s1 = state["state1"]
        qs = p.qparam[0] if p.wbit == 4 else p.qparam
        return bool(s1.dtype == torch.uint8 and s1.is_cuda and group["weight_decay"] == 0 and qs.dtype == g.dtype
                    and (p.wbit == 4 or p.shape[1] % 8 == 0))

    def _fused_quant_step(self, group, p, state):
        state["step"] += 1
        step = state["step"]
        beta1, beta2 = group["betas"]
        step_size = self._step_size(group, step)
        hyper = ops.make_adam_hyper(beta1, beta2, group["eps"], step_size)
        res, g = p.residual, p.grad
        if isinstance(g, GradientQTensor):
            g = g.get_value()                    # utils/quant.py:1064-1065
            if g.dtype != (p.qparam[0] if p.wbit == 4 else p.qparam).dtype:
                state["step"] -= 1
                return self.update_step(group, p, None, None)
        st = (state["state1"], state["qmap1"], state["absmax1"], state["state2"], state["qmap2"], state["absmax2"])
        # The step that also refreshes the residual-curve level (utils/quant.py:1107-1111): one extra read-only pass leaves
        # the sums of |exp_avg| / denom per 128 elements; the rest is a handful of operations on one value per group / row.
        # It runs BEFORE the step, like the reference's update_mu, so this step already encodes with the new level.
        if step > 250 and step % self.mu_updata_f == self.mu_updata_f - 1:
            if p.numel() % 128 != 0 or res.qshape[1] % 128 != 0:
                raise RuntimeError("residual-curve refresh needs statistics rows that are multiples of 128 elements")
            stat = ops.adam_moment_stat(g, *st, hyper)
            per = res.qshape[1]                                    # elements per statistics row: 128 (A16W4) or the row length
            sums = stat.view(-1, 1) if per == 128 else stat.view(res.qshape[0], per // 128).sum(dim=1, keepdim=True)
            optmizer_std = (sums / per).to(g.dtype) * step_size    # torch.mean(...) in the chain dtype, then * step_size
            res.update_mu(optmizer_std)
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=g.dtype, res_round_bf16=True,
                          has_residual=not res.init, mu_enc=res.mu, mu_dec=res.lock_mu)
        if p.wbit == 4:
            flat = getattr(p, "_flat_qparams", None)
            if flat is None or flat[2] is not p.qparam[0]:
                flat = p._flat_qparams = (p.qparam[0].contiguous().reshape(-1), p.qparam[1].contiguous().reshape(-1), p.qparam[0])
            ops.adam_a16w4_step(p.data, res.residual_int.view(-1), g, flat[0], flat[1], *st, hyper, o, GROUPSIZE)
            scale_col = flat[0].view(-1, 1)
        else:
            qs = p.qparam.contiguous().reshape(-1)
            ops.adam_a8w8_step(p.data.view(p.shape[0], -1), res.residual_int.view(-1), g.view(p.shape[0], -1), qs, *st, hyper, o)
            scale_col = qs.view(-1, 1)
        res._after_set_value(scale_col)
        if isinstance(p.grad, GradientQTensor):
            p.grad.zero()
        else:
            p.grad = None

    @staticmethod
    def _fused_dense_ok(group, p, state):
        if isinstance(p, (QuantTensor, FPTensor)) or not torch.is_tensor(p) or group["weight_decay"] != 0:
            return False
        g, s1, s2 = p.grad, state["state1"], state["state2"]
        return (p.is_cuda and p.dtype == torch.bfloat16 and p.data.is_contiguous() and torch.is_tensor(g)
                and g.dtype == torch.bfloat16 and g.is_cuda and g.is_contiguous() and g.shape == p.shape
                and s1.dtype == torch.bfloat16 and s1.is_cuda and s2.dtype == torch.bfloat16 and s2.is_cuda
                and s1.is_contiguous() and s2.is_contiguous())

    def _fused_dense_step(self, gindex, group, plist):
        step = self.state[plist[0]]["step"] + 1
        beta1, beta2 = group["betas"]
        hyper = ops.make_adam_hyper(beta1, beta2, group["eps"], self._step_size(group, step))
        table = self._dense_tables.setdefault(gindex, ops.DenseAdamTable())
        table.update([p.data for p in plist], [p.grad for p in plist],
                     [self.state[p]["state1"] for p in plist], [self.state[p]["state2"] for p in plist])
        ops.adam_dense_multi(table, hyper)
        for p in plist:
            self.state[p]["step"] = step
            p.grad = None

    def get_config(self, gindex, pindex, group):
        return {"betas": group["betas"], "eps": group["eps"], "weight_decay": group["weight_decay"], "lr": group["lr"],
                "block_wise": True}

    def get_state_buffer(self, pshape, pdevice, dtype=torch.float32):
        return torch.zeros(pshape, dtype=dtype, device=pdevice)

    @torch.no_grad()
    def init_state(self, group, p, gindex, pindex):
        dtype = torch.uint8 if self.obit == 8 else torch.bfloat16
        if p.numel() < 65536:
            dtype = torch.bfloat16
        state = self.state[p]
        state["step"] = 0
        shape = tuple(p.shape)
        if dtype == torch.bfloat16:
            state["state1"] = self.get_state_buffer(shape, self.statedevice, dtype=dtype)
            state["state2"] = self.get_state_buffer(shape, self.statedevice, dtype=dtype)
        else:
            state["state1"] = self.get_state_buffer(shape, self.statedevice, dtype=torch.uint8)
            state["state2"] = self.get_state_buffer(shape, self.statedevice, dtype=torch.uint8)
            n = p.numel()
            if n % 2048 == 0:
                blocks = n // 2048
            else:
                assert n % 128 == 0
                blocks = n // 128
            for k in ("absmax1", "absmax2"):
                state[k] = torch.zeros((blocks, 1), dtype=torch.float32, device=p.device)
            for k in ("qmap1", "qmap2"):
                state[k] = torch.zeros((blocks, 1), dtype=torch.float32, device=p.device) + 1e-10

    @torch.no_grad()
    def update_step(self, group, p, gindex, pindex):
        state = self.state[p]
        config = self.get_config(gindex, pindex, group)
        grad = p.grad
        if isinstance(p, QuantTensor):
            if isinstance(grad, GradientQTensor):
                grad = grad.get_value()
            if isinstance(p.residual, ResidualTensor):
                if p.wbit == 8:
                    pdata = p.residual.add((p.data * p.qparam).to(grad.dtype))
                elif p.wbit == 4:
                    pdata = p.residual.add(DeQfunc_4bit_g(p.data, p.qparam, grad.dtype))
                else:
                    assert False
            else:
                pdata = p.residual.data.to(grad.dtype)
        else:
            pdata = p.data

        if state["state1"].dtype == torch.uint8:
            exp_avg = DeQfunc_8bit_opt(state["state1"].to(grad.device), [state["qmap1"], state["absmax1"]]).to(grad.dtype)
        else:
            exp_avg = state["state1"].to(grad.device)
        if state["state2"].dtype == torch.uint8:
            s2 = DeQfunc_8bit_opt(state["state2"].to(grad.device), [state["qmap2"], state["absmax2"]])
            exp_avg_sq = (s2 * s2).to(grad.dtype)
        else:
            exp_avg_sq = (state["state2"] * state["state2"]).to(grad.device)

        beta1, beta2 = config["betas"]
        state["step"] += 1
        if config["weight_decay"] != 0:
            grad = grad.add(pdata, alpha=config["weight_decay"])
        exp_avg.mul_(beta1).add_(grad, alpha=1 - beta1)
        exp_avg_sq.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
        exp_avg_sqrt = exp_avg_sq.sqrt_()
        denom = exp_avg_sqrt.add_(group["eps"])
        bias_correction1 = 1 - beta1 ** state["step"]
        bias_correction2 = 1 - beta2 ** state["step"]
        step_size = config["lr"] * math.sqrt(bias_correction2) / bias_correction1
        pdata.addcdiv_(exp_avg, denom, value=-step_size)

        if (state["step"] > 250 and state["step"] % self.mu_updata_f == (self.mu_updata_f - 1) and hasattr(p, 'residual')
                and isinstance(p.residual, ResidualTensor)):
            optmizer_std = torch.mean((abs(exp_avg) / denom).view(p.residual.qshape), dim=1, keepdim=True) * step_size
            p.residual.update_mu(optmizer_std)

        if state["state1"].dtype == torch.uint8:
            state1, qparam = Qfunc_8bit_opt(exp_avg.float(), blocksize=len(state["absmax1"]))
            state["state1"] = state1.to(state["state1"].device)
            state["qmap1"], state["absmax1"] = qparam
        else:
            state["state1"] = exp_avg
        if state["state2"].dtype == torch.uint8:
            state2, qparam = Qfunc_8bit_opt(exp_avg_sqrt.float(), blocksize=len(state["absmax2"]))
            state["state2"] = state2.to(state["state2"].device)
            state["qmap2"], state["absmax2"] = qparam
        else:
            state["state2"] = exp_avg_sq

        if isinstance(p, QuantTensor):
            new_codes = None
            if p.wbit == 8:
                new_codes = Qfunc_8bit_res(pdata, p.residual, qscales=p.qparam)
            elif p.wbit == 4:
                new_codes = Qfunc_4bit_g_res(pdata, p.residual, qparam=p.qparam)
            if new_codes is not None:
                old = p.data
                # same values as the reference's `p.data = ...`; written into the existing storage when possible so that
                # captured CUDA graphs of the forward/backward keep reading the live codes
                if (torch.is_tensor(old) and old.is_cuda and old.dtype == new_codes.dtype and old.numel() == new_codes.numel()
                        and old.device == new_codes.device and old.is_contiguous()):
                    old.view(-1).copy_(new_codes.reshape(-1))
                else:
                    p.data = new_codes
        if isinstance(p.grad, GradientQTensor):
            p.grad.zero()
        else:
            p.grad = None
