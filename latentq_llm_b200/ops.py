"""Torch-tensor front-end of the C ABI (device memory and streams only; all arithmetic is in the
CUDA library).  Every function validates device / dtype / contiguity, allocates the outputs the
reference's Python code would allocate, and launches on torch's current stream."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from ._lib import (CODEC_NONE, CODEC_THREEFOLD, CODEC_UNIFORM16, DITHER_EXPLICIT, DITHER_HASH,  # noqa: F401
                   DITHER_PHILOX, LQ_BF16, LQ_F32, RequantOpts)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return LQ_F32
    if t.dtype == torch.bfloat16:
        return LQ_BF16
    raise TypeError(f"unsupported dtype {t.dtype} (float32 or bfloat16 expected)")


def _chk(t: torch.Tensor, name: str, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def make_opts(codec=CODEC_THREEFOLD, dither=DITHER_HASH, math_dtype=torch.bfloat16, res_round_bf16=True,
              has_residual=True, mu_enc=0, mu_dec=0, v0=0.0, seed=0, step=0, param_id=0, dither_buf=None) -> RequantOpts:
    o = RequantOpts()
    o.codec, o.dither = codec, dither
    o.math_dtype = LQ_BF16 if math_dtype == torch.bfloat16 else LQ_F32
    o.res_round_bf16, o.has_residual = int(res_round_bf16), int(has_residual)
    o.mu_enc, o.mu_dec, o.v0 = mu_enc, mu_dec, v0
    o.seed = seed & 0xFFFFFFFFFFFFFFFF
    o.stream_id = ((step & 0xFFFFFFFF) << 32) | (param_id & 0xFFFFFFFF)
    if dither_buf is not None:
        _chk(dither_buf, "dither_buf", torch.float32)
        o.dither_buf = dither_buf.data_ptr()
        o._keepalive = dither_buf      # the struct only holds the address
    return o


# ---- residual codecs (MyQuantDequant) ---------------------------------------------------------
def res3_quant(x, words, k1, b1, k2, b2, k3, v0=0.0):
    _chk(x, "x"); _chk(words, "words", torch.int32)
    assert x.numel() == 8 * words.numel()
    L.call("lq_res3_quant", _ptr(x), _dt(x), _ptr(words), words.numel(), k1, b1, k2, b2, k3, v0, _stream())


def res3_dequant(words, x, k1, b1, k2, b2, k3):
    _chk(x, "x"); _chk(words, "words", torch.int32)
    assert x.numel() == 8 * words.numel()
    L.call("lq_res3_dequant", _ptr(words), _ptr(x), _dt(x), words.numel(), k1, b1, k2, b2, k3, _stream())


def resu_quant(x, words, v0=0.0):
    _chk(x, "x"); _chk(words, "words", torch.int32)
    assert x.numel() == 8 * words.numel()
    L.call("lq_resu_quant", _ptr(x), _dt(x), _ptr(words), words.numel(), v0, _stream())


def resu_quant_s(x, words):
    _chk(x, "x"); _chk(words, "words", torch.int32)
    assert x.numel() == 8 * words.numel()
    L.call("lq_resu_quant_s", _ptr(x), _dt(x), _ptr(words), words.numel(), _stream())


def resu_dequant(words, x):
    _chk(x, "x"); _chk(words, "words", torch.int32)
    assert x.numel() == 8 * words.numel()
    L.call("lq_resu_dequant", _ptr(words), _ptr(x), _dt(x), words.numel(), _stream())


def uniform16_encode(r, noise):
    _chk(r, "r", torch.float32); _chk(noise, "noise", torch.float32)
    words = torch.empty(r.numel() // 8, dtype=torch.int32, device=r.device)
    carry = torch.empty_like(r)
    L.call("lq_uniform16_encode", _ptr(r), _ptr(noise), r.numel(), _ptr(words), _ptr(carry), _stream())
    return words, carry


def uniform16_decode(words):
    _chk(words, "words", torch.int32)
    out = torch.empty(words.numel() * 8, dtype=torch.float32, device=words.device)
    L.call("lq_uniform16_decode", _ptr(words), words.numel(), _ptr(out), _stream())
    return out


# ---- packing / dequant / qparams --------------------------------------------------------------
def pack_nibbles(codes):
    _chk(codes, "codes", torch.uint8)
    out = torch.empty(codes.numel() // 2, dtype=torch.int8, device=codes.device)
    L.call("lq_pack_nibbles", _ptr(codes), _ptr(out), codes.numel(), _stream())
    return out


def unpack_nibbles(packed):
    _chk(packed, "packed", torch.int8)
    out = torch.empty(packed.numel() * 2, dtype=torch.int8, device=packed.device)
    L.call("lq_unpack_nibbles", _ptr(packed), _ptr(out), packed.numel(), _stream())
    return out


def nibblepair_to_gptq(qweight_np, N, K):
    _chk(qweight_np, "qweight_np", torch.int8)
    out = torch.empty((K // 8, N), dtype=torch.int32, device=qweight_np.device)
    L.call("lq_nibblepair_to_gptq", _ptr(qweight_np), _ptr(out), N, K, _stream())
    return out


def gptq_to_nibblepair(qweight_gptq, N, K):
    _chk(qweight_gptq, "qweight_gptq", torch.int32)
    out = torch.empty(N * K // 2, dtype=torch.int8, device=qweight_gptq.device)
    L.call("lq_gptq_to_nibblepair", _ptr(qweight_gptq), _ptr(out), N, K, _stream())
    return out


def a16w4_dequant(qweight, scales, zeros, shape, dtype=torch.bfloat16, group=128):
    _chk(qweight, "qweight", torch.int8); _chk(scales, "scales"); _chk(zeros, "zeros", scales.dtype)
    numel = qweight.numel() * 2
    out = torch.empty(shape, dtype=dtype, device=qweight.device)
    assert out.numel() == numel and scales.numel() == numel // group
    L.call("lq_a16w4_dequant", _ptr(qweight), _ptr(scales), _ptr(zeros), _dt(scales), _ptr(out), _dt(out), numel, group,
           _stream())
    return out


def find_qparams(x, group=128, maxq=15, sym=False):
    _chk(x, "x")
    n_groups = x.numel() // group
    scales = torch.empty(n_groups, dtype=torch.float32, device=x.device)
    zeros = torch.empty_like(scales)
    L.call("lq_find_qparams", _ptr(x), _dt(x), x.numel(), group, maxq, int(sym), _ptr(scales), _ptr(zeros), _stream())
    return scales, zeros


# ---- requantize -----------------------------------------------------------------------------
def a16w4_requant(w, scales, zeros, opts: RequantOpts, group=128, codes_out=None, words_out=None):
    _chk(w, "w"); _chk(scales, "scales"); _chk(zeros, "zeros", scales.dtype)
    numel = w.numel()
    if codes_out is None:
        codes_out = torch.empty(numel // 2, dtype=torch.int8, device=w.device)
    if words_out is None and opts.codec != CODEC_NONE:
        words_out = torch.empty(numel // 8, dtype=torch.int32, device=w.device)
    L.call("lq_a16w4_requant", _ptr(w), _dt(w), _ptr(scales), _ptr(zeros), _dt(scales), numel, group, C.byref(opts),
           _ptr(codes_out), _ptr(words_out), _stream())
    return codes_out, words_out


def a16w4_fold_delta(codes, words, delta, scales, zeros, opts: RequantOpts, group=128):
    _chk(codes, "codes", torch.int8); _chk(scales, "scales"); _chk(zeros, "zeros", scales.dtype)
    if words is not None:
        _chk(words, "words", torch.int32)
    if delta is not None:
        _chk(delta, "delta")
        assert delta.numel() == codes.numel() * 2
    L.call("lq_a16w4_fold_delta", _ptr(codes), _ptr(words), _ptr(delta), 0 if delta is None else _dt(delta), _ptr(scales),
           _ptr(zeros), _dt(scales), codes.numel() * 2, group, C.byref(opts), _stream())


def a8w8_requant(w, qscales, opts: RequantOpts, codes_out=None, words_out=None):
    _chk(w, "w"); _chk(qscales, "qscales")
    rows, cols = w.shape
    if codes_out is None:
        codes_out = torch.empty((rows, cols), dtype=torch.int8, device=w.device)
    if words_out is None and opts.codec != CODEC_NONE:
        words_out = torch.empty(rows * cols // 8, dtype=torch.int32, device=w.device)
    L.call("lq_a8w8_requant", _ptr(w), _dt(w), _ptr(qscales), _dt(qscales), rows, cols, C.byref(opts), _ptr(codes_out),
           _ptr(words_out), _stream())
    return codes_out, words_out


def a8w8_fold_delta(codes, words, delta, qscales, opts: RequantOpts):
    _chk(codes, "codes", torch.int8); _chk(qscales, "qscales")
    rows, cols = codes.shape
    if delta is not None:
        _chk(delta, "delta")
    L.call("lq_a8w8_fold_delta", _ptr(codes), _ptr(words), _ptr(delta), 0 if delta is None else _dt(delta), _ptr(qscales),
           _dt(qscales), rows, cols, C.byref(opts), _stream())


def philox_dither(seed, stream_id, n_words, device, first_word=0):
    out = torch.empty(n_words * 8, dtype=torch.float32, device=device)
    L.call("lq_philox_dither", seed, stream_id, first_word, n_words, _ptr(out), _stream())
    return out


# ---- optimizer-state codec ---------------------------------------------------------------------
def opt8_quant(x, block):
    _chk(x, "x", torch.float32)
    n = x.numel()
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty((n // block, 1), dtype=torch.float32, device=x.device)
    tmax = torch.empty_like(scale)
    L.call("lq_opt8_quant", _ptr(x), n, block, _ptr(q), _ptr(scale), _ptr(tmax), _stream())
    return q, scale, tmax


def opt8_dequant(q, block, scale, tmax):
    _chk(q, "q", torch.uint8); _chk(scale, "scale", torch.float32); _chk(tmax, "tmax", torch.float32)
    x = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    L.call("lq_opt8_dequant", _ptr(q), q.numel(), block, _ptr(scale), _ptr(tmax), _ptr(x), _stream())
    return x


# ---- activation quantizers ---------------------------------------------------------------------
# ---- fused optimizer step -------------------------------------------------------------------------
def make_adam_hyper(beta1, beta2, eps, step_size) -> "L.AdamHyper":
    """Python doubles -> the fp32 scalars torch's bf16/fp32 elementwise ops would compute with."""
    h = L.AdamHyper()
    h.beta1, h.beta2 = beta1, beta2
    h.one_minus_beta1, h.one_minus_beta2 = 1 - beta1, 1 - beta2
    h.eps, h.neg_step_size = eps, -step_size
    return h


def adam_a16w4_step(codes, words, grad, scales, zeros, state1, scale1, tmax1, state2, scale2, tmax2,
                    hyper, opts: RequantOpts, group=128):
    """In place on codes / words / both states and their block parameters."""
    _chk(codes, "codes", torch.int8); _chk(words, "words", torch.int32); _chk(grad, "grad")
    _chk(scales, "scales"); _chk(zeros, "zeros", scales.dtype)
    _chk(state1, "state1", torch.uint8); _chk(state2, "state2", torch.uint8)
    for t, nm in ((scale1, "scale1"), (tmax1, "tmax1"), (scale2, "scale2"), (tmax2, "tmax2")):
        _chk(t, nm, torch.float32)
    n = grad.numel()
    assert codes.numel() * 2 == n and words.numel() * 8 == n and state1.numel() == n and state2.numel() == n
    blocks = scale1.numel()
    assert tmax1.numel() == blocks and scale2.numel() == blocks and tmax2.numel() == blocks and n % blocks == 0
    L.check("lq_adam_a16w4_step", L.lib.lq_adam_a16w4_step(
        _ptr(codes), _ptr(words), _ptr(grad), _dt(grad), _ptr(scales), _ptr(zeros), _dt(scales), n, group,
        _ptr(state1), _ptr(scale1), _ptr(tmax1), _ptr(state2), _ptr(scale2), _ptr(tmax2), n // blocks,
        C.byref(hyper), C.byref(opts), _stream()))


def adam_a8w8_step(codes, words, grad, qscales, state1, scale1, tmax1, state2, scale2, tmax2, hyper, opts: RequantOpts):
    """MyAdam.update_step for one A8W8 weight (int8 codes [rows, cols], one scale per row), in place."""
    _chk(codes, "codes", torch.int8); _chk(words, "words", torch.int32); _chk(grad, "grad"); _chk(qscales, "qscales", grad.dtype)
    _chk(state1, "state1", torch.uint8); _chk(state2, "state2", torch.uint8)
    rows, cols = grad.shape
    n = rows * cols
    assert codes.numel() == n and words.numel() * 8 == n and qscales.numel() == rows and state1.numel() == n and state2.numel() == n
    blocks = scale1.numel()
    L.check("lq_adam_a8w8_step", L.lib.lq_adam_a8w8_step(
        _ptr(codes), _ptr(words), _ptr(grad), _dt(grad), _ptr(qscales), _dt(qscales), rows, cols,
        _ptr(state1), _ptr(scale1), _ptr(tmax1), _ptr(state2), _ptr(scale2), _ptr(tmax2), n // blocks,
        C.byref(hyper), C.byref(opts), _stream()))


def adam_moment_stat(grad, state1, scale1, tmax1, state2, scale2, tmax2, hyper):
    """Sums of |exp_avg| / denom per 128 elements for the step about to be taken (utils/quant.py:1107-1111)."""
    _chk(grad, "grad"); _chk(state1, "state1", torch.uint8); _chk(state2, "state2", torch.uint8)
    n = grad.numel()
    out = torch.empty(n // 128, dtype=torch.float32, device=grad.device)
    L.check("lq_adam_moment_stat", L.lib.lq_adam_moment_stat(
        _ptr(grad), _dt(grad), n, _ptr(state1), _ptr(scale1), _ptr(tmax1), _ptr(state2), _ptr(scale2), _ptr(tmax2),
        n // scale1.numel(), C.byref(hyper), _ptr(out), _stream()))
    return out


class DenseAdamTable:
    """Device-resident table of small dense bf16 parameters for `adam_dense_multi` (rebuilt only when an address
    changes: parameter data, arena gradient views and in-place states keep theirs from step to step)."""

    def __init__(self):
        self.key, self.dev, self.n, self.max_numel, self.keep = None, None, 0, 0, None

    def update(self, params, grads, states1, states2):
        key = tuple((p.data_ptr(), g.data_ptr(), a.data_ptr(), b.data_ptr(), p.numel())
                    for p, g, a, b in zip(params, grads, states1, states2))
        if key != self.key:
            arr = (L.DenseSlot * len(key))()
            for i, (pp, gp, ap, bp, n) in enumerate(key):
                arr[i].param, arr[i].grad, arr[i].state1, arr[i].state2, arr[i].numel = pp, gp, ap, bp, n
            host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
            self.dev = host.to(params[0].device)
            self.key, self.n = key, len(key)
            self.max_numel = max(k[4] for k in key)
        self.keep = (list(params), list(grads), list(states1), list(states2))


def adam_dense_multi(table: DenseAdamTable, hyper):
    if table.n == 0:
        return
    L.check("lq_adam_dense_multi", L.lib.lq_adam_dense_multi(_ptr(table.dev), table.n, table.max_numel,
                                                             C.byref(hyper), _stream()))


def act_quant_per_token(x):
    _chk(x, "x", torch.bfloat16)
    M, K = x.shape
    x8 = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty(M, dtype=torch.float32, device=x.device)
    L.call("lq_act_quant_per_token", _ptr(x), M, K, _ptr(x8), _ptr(s), _stream())
    return x8, s


def act_quant_per_tensor(x):
    _chk(x, "x", torch.bfloat16)
    x8 = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    clampv = torch.empty(1, dtype=torch.float32, device=x.device)
    L.call("lq_act_quant_per_tensor", _ptr(x), x.numel(), _ptr(clampv), _ptr(x8), _stream())
    return x8, clampv


# ---- GEMMs --------------------------------------------------------------------------------------
_workspaces: dict = {}


_ws_need: dict = {}


def _workspace(kind, M, N, K, device):
    need = _ws_need.get((kind, M, N, K))
    if need is None:
        need = _ws_need[(kind, M, N, K)] = int(L.lib.lq_gemm_workspace_bytes(kind, M, N, K))
    if need == 0:
        return None, 0
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws, ws.numel()


def gemm_a16w4_fwd(x, qweight, scales, zeros, bias, N, K, group=128, out=None):
    _chk(x, "x", torch.bfloat16); _chk(qweight, "qweight", torch.int8)
    _chk(scales, "scales", torch.bfloat16); _chk(zeros, "zeros", torch.bfloat16)
    M = x.shape[0]
    assert x.shape[1] == K and qweight.numel() * 2 == N * K
    if bias is not None:
        _chk(bias, "bias", torch.bfloat16)
    y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ws, nb = _workspace(L.GEMM_A16W4_FWD, M, N, K, x.device)
    L.call("lq_gemm_a16w4_fwd", _ptr(x), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(bias), _ptr(y), M, N, K, group,
           _ptr(ws), nb, _stream())
    return y


def gemm_a16w4_dgrad(dy, qweight, scales, zeros, N, K, group=128, out=None):
    _chk(dy, "dy", torch.bfloat16); _chk(qweight, "qweight", torch.int8)
    _chk(scales, "scales", torch.bfloat16); _chk(zeros, "zeros", torch.bfloat16)
    M = dy.shape[0]
    assert dy.shape[1] == N and qweight.numel() * 2 == N * K
    dx = out if out is not None else torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
    ws, nb = _workspace(L.GEMM_A16W4_DGRAD, M, N, K, dy.device)
    L.call("lq_gemm_a16w4_dgrad", _ptr(dy), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(dx), M, N, K, group, _ptr(ws), nb,
           _stream())
    return dx


def gemm_wgrad(dy, x, dw=None, accumulate=False):
    """dw[N, K] (+)= dy[M, N]^T · x[M, K] (utils/quant.py:141-142): the weight gradient of a quantized linear, written
    (or accumulated, one rounding of the fp32 sum) straight into `dw`, e.g. a view of the gradient arena."""
    _chk(dy, "dy", torch.bfloat16); _chk(x, "x", torch.bfloat16)
    M, N = dy.shape
    K = x.shape[1]
    assert x.shape[0] == M
    if dw is None:
        assert not accumulate
        dw = torch.empty((N, K), dtype=torch.bfloat16, device=dy.device)
    else:
        _chk(dw, "dw", torch.bfloat16)
        assert tuple(dw.shape) == (N, K)
    L.call("lq_gemm_wgrad", _ptr(dy), _ptr(x), _ptr(dw), M, N, K, int(accumulate), _stream())
    return dw


def gemm_a8w8(x8, w8, row_scale=None, col_scale=None, alpha=1.0, bias=None, want_acc=False):
    _chk(x8, "x8", torch.int8); _chk(w8, "w8", torch.int8)
    M, K = x8.shape
    N = w8.shape[0]
    assert w8.shape[1] == K
    for t, nm in ((row_scale, "row_scale"), (col_scale, "col_scale")):
        if t is not None:
            _chk(t, nm, torch.float32)
    if bias is not None:
        _chk(bias, "bias", torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x8.device)
    acc = torch.empty((M, N), dtype=torch.int32, device=x8.device) if want_acc else None
    ws, nb = _workspace(L.GEMM_A8W8, M, N, K, x8.device)
    L.call("lq_gemm_a8w8", _ptr(x8), _ptr(w8), _ptr(row_scale), _ptr(col_scale), float(alpha), _ptr(bias), _ptr(y), _ptr(acc),
           M, N, K, _ptr(ws), nb, _stream())
    return (y, acc) if want_acc else y


class decode_chain:
    """Context manager: launches inside it form a decode chain (every kernel consumes its predecessor's output, the
    weights are constant), so the decode kernels may be started while their predecessor is still running; they read what
    the predecessor wrote only after it has completed.  Outside such a block a forward right after an optimizer step is
    safe: nothing is read early."""

    def __enter__(self):
        self.old = L.lib.lq_decode_chain(1)
        return self

    def __exit__(self, *exc):
        L.lib.lq_decode_chain(self.old)
        return False


# ---- decode-side operations of a Llama-architecture layer ------------------------------------------
def add_rmsnorm(h, delta, gamma, eps, out=None, hf_rounding=True):
    """h [M, K] += delta (in place, when given); returns RMSNorm(h) * gamma (PTQ/quant/triton_norm.py:7-39)."""
    _chk(h, "h", torch.bfloat16); _chk(gamma, "gamma", torch.bfloat16)
    if delta is not None:
        _chk(delta, "delta", torch.bfloat16)
        assert delta.shape == h.shape
    M, K = h.shape
    y = out if out is not None else torch.empty_like(h)
    L.call("lq_add_rmsnorm", _ptr(h), _ptr(delta), _ptr(gamma), float(eps), _ptr(y), M, K, int(hf_rounding), _stream())
    return y


def gemm_a16w4_fwd_rmsnorm(h, delta, gamma, eps, h_out, qweight, scales, zeros, N, K, group=128, out=None, silu_pair=False,
                           hf_rounding=True):
    """y = (RMSNorm(h + delta) * gamma) · deq(Wq)^T in ONE launch for decode-sized token counts (at most two tokens,
    K = 4096, group 128): the residual add and the norm happen in the GEMM kernel's token staging, bit for bit as
    `add_rmsnorm` computes them.  `h_out` (a buffer other than `h`) receives h + delta when `delta` is given.  With
    `silu_pair` the weight holds gate | up (N = 2 I rows) and the result is silu(gate) * up [M, I].
    Returns None when the shape has no fused kernel: call `add_rmsnorm` and the GEMM separately then."""
    _chk(h, "h", torch.bfloat16); _chk(gamma, "gamma", torch.bfloat16); _chk(qweight, "qweight", torch.int8)
    M = h.shape[0]
    if delta is not None:
        _chk(delta, "delta", torch.bfloat16); _chk(h_out, "h_out", torch.bfloat16)
        assert delta.shape == h.shape == h_out.shape and h_out.data_ptr() != h.data_ptr()
    n_out = N // 2 if silu_pair else N
    y = out if out is not None else torch.empty((M, n_out), dtype=torch.bfloat16, device=h.device)
    rc = L.lib.lq_gemm_a16w4_fwd_rmsnorm(_ptr(h), _ptr(delta), _ptr(gamma), float(eps), int(hf_rounding), _ptr(h_out),
                                         _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(y), M, N, K, group, int(silu_pair),
                                         _stream())
    if rc == L.LQ_EUNSUPPORTED:
        return None
    L.check("lq_gemm_a16w4_fwd_rmsnorm", rc)
    return y


def gemm_a16w4_fwd_qkv_rope(x, qweight, scales, zeros, positions, inv_freq, k_cache, v_cache, Hq, Hkv, hd, K, group=128, out=None,
                            tokens_per_seq=1, hf_rounding=True, norm=None):
    """Decode-sized fused q|k|v projection with the rotary embedding and the KV-cache write as its epilogue: leaves what
    `gemm_a16w4_fwd` followed by `rope_kv_store` leaves (q rotated in the returned [M, (Hq + 2 Hkv) hd] buffer, rotated k
    and v in the caches), in one launch.  `norm=(h, delta, gamma, eps, h_out)` computes the tokens as
    RMSNorm(h + delta) * gamma in the same launch (`x` is ignored; see `gemm_a16w4_fwd_rmsnorm`).
    Returns None when the shape has no fused kernel."""
    _chk(qweight, "qweight", torch.int8); _chk(positions, "positions", torch.int64); _chk(inv_freq, "inv_freq", torch.float32)
    _chk(k_cache, "k_cache", torch.bfloat16); _chk(v_cache, "v_cache", torch.bfloat16)
    h = delta = gamma = h_out = None
    eps = 0.0
    if norm is not None:
        h, delta, gamma, eps, h_out = norm
        _chk(h, "h", torch.bfloat16); _chk(gamma, "gamma", torch.bfloat16)
        if delta is not None:
            _chk(delta, "delta", torch.bfloat16); _chk(h_out, "h_out", torch.bfloat16)
            assert delta.shape == h.shape == h_out.shape and h_out.data_ptr() != h.data_ptr()
        M = h.shape[0]
    else:
        _chk(x, "x", torch.bfloat16)
        M = x.shape[0]
    N = (Hq + 2 * Hkv) * hd
    max_len = k_cache.shape[2]
    assert positions.numel() == M and inv_freq.numel() == hd // 2 and k_cache.shape == v_cache.shape and k_cache.shape[3] == hd
    y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=qweight.device)
    rc = L.lib.lq_gemm_a16w4_fwd_qkv_rope(_ptr(None if norm is not None else x), _ptr(h), _ptr(delta), _ptr(gamma), float(eps),
                                          _ptr(h_out), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(y), _ptr(positions),
                                          _ptr(inv_freq), _ptr(k_cache), _ptr(v_cache), M, Hq, Hkv, hd, K, group, max_len,
                                          tokens_per_seq, int(hf_rounding), _stream())
    if rc == L.LQ_EUNSUPPORTED:
        return None
    L.check("lq_gemm_a16w4_fwd_qkv_rope", rc)
    return y


def argmax_embed(logits, tok, positions=None, embed=None, h=None):
    """Greedy step end in one launch: tok[b] = argmax(logits[b]) (first maximum, like torch.argmax); positions += 1 and
    h[b] = embed[tok[b]] when given (generate.py:150-190 drives HF's loop, which does these as separate ops)."""
    assert logits.dim() == 2 and logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    _chk(tok, "tok", torch.int64)
    B, V = logits.shape
    D = 0
    if embed is not None:
        _chk(embed, "embed", torch.bfloat16); _chk(h, "h", torch.bfloat16)
        D = embed.shape[1]
        assert h.shape == (B, D)
    if positions is not None:
        _chk(positions, "positions", torch.int64)
    L.call("lq_argmax_embed", _ptr(logits), logits.stride(0), B, V, _ptr(embed), D, _ptr(tok), _ptr(positions), _ptr(h), _stream())
    return tok


def rope_kv_store(qkv, positions, inv_freq, k_cache, v_cache, Hq, Hkv, hd, tokens_per_seq=1, hf_rounding=True):
    """RoPE on the q and k heads of qkv [M, (Hq + 2 Hkv) hd] (q in place); rotated k and v go into the caches
    [batch, Hkv, max_len, hd] at positions[m] (PTQ/quant/fused_attn.py:8-58)."""
    _chk(qkv, "qkv", torch.bfloat16); _chk(positions, "positions", torch.int64); _chk(inv_freq, "inv_freq", torch.float32)
    _chk(k_cache, "k_cache", torch.bfloat16); _chk(v_cache, "v_cache", torch.bfloat16)
    M = qkv.shape[0]
    assert qkv.shape[1] == (Hq + 2 * Hkv) * hd and positions.numel() == M and inv_freq.numel() == hd // 2
    assert k_cache.shape == v_cache.shape and k_cache.shape[1] == Hkv and k_cache.shape[3] == hd
    L.call("lq_rope_kv_store", _ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(k_cache), _ptr(v_cache), M, tokens_per_seq,
           Hq, Hkv, hd, k_cache.shape[2], int(hf_rounding), _stream())


_attn_ws: dict = {}


def decode_attention(qkv, positions, k_cache, v_cache, Hq, Hkv, hd, scale=None, out=None):
    """One query token per sequence against the cache: q = first Hq*hd columns of qkv [B, ...]; keys 0..positions[b]."""
    _chk(qkv, "qkv", torch.bfloat16); _chk(positions, "positions", torch.int64)
    B, max_len = qkv.shape[0], k_cache.shape[2]
    y = out if out is not None else torch.empty((B, Hq * hd), dtype=torch.bfloat16, device=qkv.device)
    need = int(L.lib.lq_decode_attention_workspace_bytes(B, Hq, hd, max_len))
    # one workspace per shape and stream: the ticket counters sit behind the partial results, at an offset that depends on
    # the shape, and must be zero when a call starts (every call leaves them zero)
    key = (qkv.device.index, torch.cuda.current_stream().cuda_stream, B, Hq, hd, max_len)
    ws = _attn_ws.get(key)
    if ws is None:
        ws = _attn_ws[key] = torch.zeros(max(need, 1), dtype=torch.uint8, device=qkv.device)
    L.call("lq_decode_attention", _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(y), B, Hq, Hkv,
           hd, max_len, float(scale if scale is not None else hd ** -0.5), _ptr(ws), ws.numel(), _stream())
    return y


def silu_mul(gate_up, out=None, hf_rounding=True):
    """silu(gate_up[:, :I]) * gate_up[:, I:] (PTQ/quant/fused_mlp.py:84-168)."""
    _chk(gate_up, "gate_up", torch.bfloat16)
    M, I2 = gate_up.shape
    y = out if out is not None else torch.empty((M, I2 // 2), dtype=torch.bfloat16, device=gate_up.device)
    L.call("lq_silu_mul", _ptr(gate_up), _ptr(y), M, I2 // 2, int(hf_rounding), _stream())
    return y


# ---- 8-bit gradient accumulator (GradientQTensor, utils/quant.py:846-921) ---------------------------
def gradq_accumulate(fdata, qdata, scale, first, opts):
    """set_value (first) / add_ of the 8-bit stochastic gradient accumulator, in place on qdata [rows, cols] int8 and
    scale [rows] (fdata's dtype)."""
    _chk(fdata, "fdata"); _chk(qdata, "qdata", torch.int8); _chk(scale, "scale", fdata.dtype)
    rows, cols = fdata.shape
    assert qdata.shape == fdata.shape and scale.numel() == rows
    L.call("lq_gradq_accumulate", _ptr(fdata), _dt(fdata), rows, cols, _ptr(qdata), _ptr(scale), int(first), C.byref(opts), _stream())


def gradq_dequant(qdata, scale, out=None):
    _chk(qdata, "qdata", torch.int8); _chk(scale, "scale")
    rows, cols = qdata.shape
    y = out if out is not None else torch.empty((rows, cols), dtype=scale.dtype, device=qdata.device)
    L.call("lq_gradq_dequant", _ptr(qdata), _ptr(scale), _dt(scale), rows, cols, _ptr(y), _stream())
    return y


def gemm_a16w4_fwd_silu(x, qweight, scales, zeros, I, K, group=128, out=None, gate_up=None, hf_rounding=True):
    """act[M, I] = silu(x·Wgate^T) * (x·Wup^T) for a fused gate | up weight of 2*I rows (PTQ/quant/fused_mlp.py:84-168).
    Decode-sized token counts take ONE launch (the epilogue of the decode GEMM); larger ones run the GEMM into `gate_up`
    [M, 2I] (allocated if not given) and `silu_mul`."""
    _chk(x, "x", torch.bfloat16); _chk(qweight, "qweight", torch.int8)
    M = x.shape[0]
    y = out if out is not None else torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
    if M <= 16 and K % 256 == 0 and group in (128, 256) and I % 8 == 0:
        rc = L.lib.lq_gemm_a16w4_fwd_silu(_ptr(x), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(y), M, I, K, group,
                                          int(hf_rounding), _stream())
        if rc != L.LQ_EUNSUPPORTED:
            L.check("lq_gemm_a16w4_fwd_silu", rc)
            return y
    gu = gate_up if gate_up is not None else torch.empty((M, 2 * I), dtype=torch.bfloat16, device=x.device)
    gemm_a16w4_fwd(x, qweight, scales, zeros, None, 2 * I, K, group, out=gu)
    return silu_mul(gu, out=y, hf_rounding=hf_rounding)
