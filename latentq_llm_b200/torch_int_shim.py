"""Stand-in for `torch_int._CUDA` (github.com/FWkey/torch-int-bf16, un-vendored by the reference; imported at
utils/quant.py:108 and PTQ/quant/quant_linear.py:577).  Same call shape:

    linear_a8_w8_bbf16_obf16(x_i8[M,K], w_i8[N,K], bias_bf16[N], alpha) -> bf16[M,N] = alpha * (x · wᵀ)_int32 + bias

backed by the tcgen05 `kind::i8` GEMM of liblatentq.  `install()` registers this module under the name
`torch_int._CUDA` so the reference's import statement resolves to it.
"""
from __future__ import annotations

import sys
import types

import torch

from . import ops


def _alpha(alpha):
    return float(alpha.item()) if torch.is_tensor(alpha) else float(alpha)


def linear_a8_w8_bbf16_obf16(input8, weight8, bias, alpha):
    b = None if bias is None else bias.reshape(-1).to(torch.bfloat16).contiguous()
    return ops.gemm_a8w8(input8.contiguous(), weight8.contiguous(), None, None, _alpha(alpha), b)


def linear_a8_w8_bfp32_ofp32(input8, weight8, bias, alpha):
    """fp32 bias / fp32 output variant: the exact int32 accumulators scaled in fp32."""
    _, acc = ops.gemm_a8w8(input8.contiguous(), weight8.contiguous(), None, None, 1.0, None, want_acc=True)
    out = acc.float() * _alpha(alpha)
    return out if bias is None else out + bias.reshape(1, -1).float()


def linear_a8_w8_bfp16_ofp16(input8, weight8, bias, alpha):
    return linear_a8_w8_bfp32_ofp32(input8, weight8, bias, alpha).half()


def install():
    pkg = sys.modules.setdefault("torch_int", types.ModuleType("torch_int"))
    mod = types.ModuleType("torch_int._CUDA")
    for f in (linear_a8_w8_bbf16_obf16, linear_a8_w8_bfp32_ofp32, linear_a8_w8_bfp16_ofp16):
        setattr(mod, f.__name__, f)
    pkg._CUDA = mod
    sys.modules["torch_int._CUDA"] = mod
    return mod
