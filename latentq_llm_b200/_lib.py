"""ctypes binding of liblatentq.so (the C ABI declared in include/latentq.h).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "liblatentq.so")

LQ_OK, LQ_EINVAL, LQ_EUNSUPPORTED, LQ_ECUDA, LQ_ETIMEOUT, LQ_EWORKSPACE = 0, -1, -2, -3, -4, -5
LQ_F32, LQ_BF16 = 0, 1
CODEC_NONE, CODEC_UNIFORM16, CODEC_THREEFOLD = 0, 1, 2
DITHER_HASH, DITHER_EXPLICIT, DITHER_PHILOX = 0, 1, 2
GEMM_A16W4_FWD, GEMM_A16W4_DGRAD, GEMM_A8W8 = 0, 1, 2


class RequantOpts(C.Structure):
    """Mirror of `lq_requant_opts`."""
    _fields_ = [("codec", C.c_int32), ("dither", C.c_int32), ("math_dtype", C.c_int32),
                ("res_round_bf16", C.c_int32), ("has_residual", C.c_int32),
                ("mu_enc", C.c_int32), ("mu_dec", C.c_int32), ("v0", C.c_float),
                ("seed", C.c_uint64), ("stream_id", C.c_uint64), ("dither_buf", C.c_void_p)]


class AdamHyper(C.Structure):
    """Mirror of `lq_adam_hyper`."""
    _fields_ = [("beta1", C.c_float), ("beta2", C.c_float), ("one_minus_beta1", C.c_float),
                ("one_minus_beta2", C.c_float), ("eps", C.c_float), ("neg_step_size", C.c_float)]


class DenseSlot(C.Structure):
    """Mirror of `lq_dense_slot`."""
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p), ("state1", C.c_void_p), ("state2", C.c_void_p),
                ("numel", C.c_int64)]


class LatentQError(RuntimeError):
    def __init__(self, fn, status, detail=""):
        self.status = status
        super().__init__(f"{fn} failed with status {status} ({detail})")


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m latentq_llm_b200.build` "
        "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these kernels.")

lib = C.CDLL(LIB_PATH)

_p, _i, _i64, _f, _u64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint64, C.c_size_t
_OPTS = C.POINTER(RequantOpts)
_HYPER = C.POINTER(AdamHyper)

# name -> argtypes; every function returns int except the ones listed in _RESTYPE.
SIGNATURES = {
    "lq_version": [],
    "lq_decode_chain": [_i],
    "lq_status_string": [_i],
    "lq_last_cuda_error": [],
    "lq_res3_quant": [_p, _i, _p, _i64, _i, _f, _i, _f, _i, _f, _p],
    "lq_res3_dequant": [_p, _p, _i, _i64, _i, _f, _i, _f, _i, _p],
    "lq_resu_quant": [_p, _i, _p, _i64, _f, _p],
    "lq_resu_quant_s": [_p, _i, _p, _i64, _p],
    "lq_resu_dequant": [_p, _p, _i, _i64, _p],
    "lq_uniform16_encode": [_p, _p, _i64, _p, _p, _p],
    "lq_uniform16_decode": [_p, _i64, _p, _p],
    "lq_pack_nibbles": [_p, _p, _i64, _p],
    "lq_unpack_nibbles": [_p, _p, _i64, _p],
    "lq_nibblepair_to_gptq": [_p, _p, _i64, _i64, _p],
    "lq_gptq_to_nibblepair": [_p, _p, _i64, _i64, _p],
    "lq_a16w4_dequant": [_p, _p, _p, _i, _p, _i, _i64, _i, _p],
    "lq_find_qparams": [_p, _i, _i64, _i, _i, _i, _p, _p, _p],
    "lq_a16w4_requant": [_p, _i, _p, _p, _i, _i64, _i, _OPTS, _p, _p, _p],
    "lq_a16w4_fold_delta": [_p, _p, _p, _i, _p, _p, _i, _i64, _i, _OPTS, _p],
    "lq_a8w8_requant": [_p, _i, _p, _i, _i64, _i64, _OPTS, _p, _p, _p],
    "lq_a8w8_fold_delta": [_p, _p, _p, _i, _p, _i, _i64, _i64, _OPTS, _p],
    "lq_fold_fallback_words": [_i, _p],
    "lq_philox_dither": [_u64, _u64, _i64, _i64, _p, _p],
    "lq_opt8_quant": [_p, _i64, _i, _p, _p, _p, _p],
    "lq_opt8_dequant": [_p, _i64, _i, _p, _p, _p, _p],
    "lq_adam_a16w4_step": [_p, _p, _p, _i, _p, _p, _i, _i64, _i, _p, _p, _p, _p, _p, _p, _i, _HYPER, _OPTS, _p],
    "lq_adam_dense_multi": [_p, _i, _i64, _HYPER, _p],
    "lq_adam_moment_stat": [_p, _i, _i64, _p, _p, _p, _p, _p, _p, _i, _HYPER, _p, _p],
    "lq_adam_a8w8_step": [_p, _p, _p, _i, _p, _i, _i64, _i64, _p, _p, _p, _p, _p, _p, _i, _HYPER, _OPTS, _p],
    "lq_gradq_accumulate": [_p, _i, _i64, _i64, _p, _p, _i, _OPTS, _p],
    "lq_gradq_dequant": [_p, _p, _i, _i64, _i64, _p, _p],
    "lq_act_quant_per_token": [_p, _i64, _i64, _p, _p, _p],
    "lq_act_quant_per_tensor": [_p, _i64, _p, _p, _p],
    "lq_gemm_workspace_bytes": [_i, _i64, _i64, _i64],
    "lq_gemm_a16w4_fwd": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _p, _sz, _p],
    "lq_gemm_a16w4_dgrad": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _p, _sz, _p],
    "lq_gemm_device_status": [_i],
    "lq_gemm_profile": [_i, _p],
    "lq_gemm_a16w4_fwd_static_max_bytes": [],
    "lq_gemm_a16w4_fwd_static": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _p],
    "lq_gemm_a16w4_fwd_static_peek": [_p, _sz, _sz],
    "lq_gemm_a8w8": [_p, _p, _p, _p, _f, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p],
    "lq_mma_issue_rate": [_i, _i, _i, _i, _i, _i, _p, _p],
    "lq_gemm_a16w4_fwd_rmsnorm": [_p, _p, _p, _f, _i, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _i, _p],
    "lq_gemm_a16w4_fwd_qkv_rope": [_p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i64, _i, _i64, _i, _i, _p],
    "lq_gemm_wgrad": [_p, _p, _p, _i64, _i64, _i64, _i, _p],
    "lq_argmax_embed": [_p, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _p],
    "lq_add_rmsnorm": [_p, _p, _p, _f, _p, _i64, _i64, _i, _p],
    "lq_rope_kv_store": [_p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i64, _i, _p],
    "lq_decode_attention_workspace_bytes": [_i64, _i, _i, _i64],
    "lq_decode_attention": [_p, _i64, _p, _p, _p, _p, _i64, _i, _i, _i, _i64, _f, _p, _sz, _p],
    "lq_silu_mul": [_p, _p, _i64, _i64, _i, _p],
    "lq_gemm_a16w4_fwd_silu": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i, _i, _p],
}
_RESTYPE = {"lq_status_string": C.c_char_p, "lq_last_cuda_error": C.c_char_p, "lq_gemm_workspace_bytes": C.c_size_t,
            "lq_gemm_a16w4_fwd_static_max_bytes": C.c_size_t, "lq_decode_attention_workspace_bytes": C.c_size_t}

for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = header and library disagree
    _fn.argtypes = _args
    _fn.restype = _RESTYPE.get(_name, C.c_int)


def check(fn_name: str, status: int) -> None:
    if status != LQ_OK:
        detail = lib.lq_status_string(status).decode()
        if status == LQ_ECUDA:
            detail += ": " + lib.lq_last_cuda_error().decode()
        raise LatentQError(fn_name, status, detail)


def call(fn_name: str, *args) -> None:
    check(fn_name, getattr(lib, fn_name)(*args))
