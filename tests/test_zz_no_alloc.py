"""The allocation-free forward GEMM (`lq_gemm_a16w4_fwd_static`) against the oracle and the workspace variant.

Some users of this library cannot allocate device memory where they call it: they run under a
framework that owns the whole device heap, or in a serving loop where an allocation's device-wide
synchronisation is not acceptable.  For them the split-K partial sums live in an array built into
the library.  This test drives the entry point through the C ABI exactly as such a caller would
(no workspace argument) on shapes whose plan really hands partial sums through the array — the
tensor-core route (M > 16) and the decode route of group size 64 — twice in a row per route, the second call smaller than the
first so that the first call's partial sums lie underneath it.  Each result is compared with the
CPU oracle and with `lq_gemm_a16w4_fwd`; the array itself is read back to show that the launch
wrote its partial sums there.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes as C
import threading

import numpy as np
import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu
RTOL = 1e-2   # the tolerance the other GEMM tests use


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _layer(N, K, group, seed):
    rng = np.random.default_rng(seed)
    w = orc.bf16_round((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    s, z = orc.find_qparams(w, group, 15, False)
    s, z = orc.bf16_round(s), orc.bf16_round(z)
    codes, _, _ = orc.a16w4_requant(s, z, w=w, group=group, codec=orc.CODEC_NONE, math_bf16=True)
    bias = orc.bf16_round((rng.standard_normal(N) * 0.1).astype(np.float32))
    return rng, codes, s, z, bias


def _call_static(lib, x, codes, s, z, bias, M, N, K, group):
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.lq_gemm_a16w4_fwd_static(_ptr(x), _ptr(codes), _ptr(s), _ptr(z), _ptr(bias), _ptr(got), M, N, K, group, stream)
    assert rc == 0, (rc, lib.lq_last_cuda_error())
    torch.cuda.synchronize()
    assert lib.lq_gemm_device_status(1) == 0
    return got


# (group, (first M, second M), balanced plan?, where partial sums of token 0 (and 1) land in the array):
#  - group 128, M > 16, whole-tile plan: the tensor-core kernel with four K-splits, partial sums laid out
#    [split][token][column]: 64 floats from 0 = split 0 of output (0, 0..63)
#  - the same in the kernel's balanced mode (forced; by itself the planner takes it for larger shapes): the owner of a
#    128-column tile computes k-blocks 0..8, helper CTAs the rest in pieces of four; the first helper's sums
#    (k = 576..831) go to part 1 of tile 0, slots laid out [tile][part][lane quarter][token][32 weight rows]:
#    64 floats from there = outputs (0, 0..31) and (1, 0..31)
#  - group 64, M <= 16: the decode kernel with four K-splits, partial sums laid out [split][token][column]
@pytest.mark.parametrize("group,Ms,balanced,peek_at", [(128, (64, 24), False, 0), (128, (64, 24), True, 4 * 64 * 32), (64, (16, 5), False, 0)])
def test_static_scratch_forward_twice_against_oracle(group, Ms, balanced, peek_at, monkeypatch):
    monkeypatch.setenv("LQ_GEMM_BALANCE", "1" if balanced else "0")
    from latentq_llm_b200 import _lib, ops
    lib = _lib.lib
    N, K = 512, 1024
    assert lib.lq_gemm_a16w4_fwd_static_max_bytes() == 8 << 20
    rng, codes_h, s_h, z_h, bias_h = _layer(N, K, group, seed=2024 + group)
    codes = torch.from_numpy(codes_h).cuda()
    s, z = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in (s_h, z_h))
    bias = torch.from_numpy(bias_h).cuda().to(torch.bfloat16)
    poison = np.full(64, 12345.0, np.float32)
    for call, M in enumerate(Ms):
        x_h = orc.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
        x = torch.from_numpy(x_h).cuda().to(torch.bfloat16)
        got = _call_static(lib, x, codes, s, z, bias, M, N, K, group)
        assert not torch.isnan(got.float()).any()
        ref = orc.gemm_a16w4(x_h, codes_h, s_h, z_h, N, K, group=group, bias=bias_h)
        err = np.abs(got.float().cpu().numpy().astype(np.float64) - ref).max() / np.abs(ref).max()
        assert err <= RTOL, (group, call, err)
        ops._ws_need.clear()                               # (the workspace size is cached per shape; the plan just changed)
        want = ops.gemm_a16w4_fwd(x, codes, s, z, bias, N, K, group=group)
        assert torch.equal(got, want), "static-scratch and workspace variants run the same kernels on the same plan"
        # the launch wrote fp32 partial sums into the built-in array: one K-slice of output (0, 0..63) differs from
        # what the previous call left there, is finite, and is only PART of the result (K really was split)
        part = np.empty(64, np.float32)
        assert lib.lq_gemm_a16w4_fwd_static_peek(part.ctypes.data_as(C.c_void_p), peek_at, 64) == 0
        assert np.isfinite(part).all() and not np.array_equal(part, poison)
        full = ref[0, :64] - bias_h[:64]
        if balanced:
            full = np.concatenate([ref[0, :32] - bias_h[:32], ref[1, :32] - bias_h[:32]])
        assert np.abs(part - full).max() > 0.05 * np.abs(full).max()
        poison = part.copy()


def test_static_scratch_from_a_thread_without_a_context():
    """A fresh host thread has no current CUDA context: the entry point has to bind the operands' device before it
    looks up the array's address."""
    from latentq_llm_b200 import _lib
    lib = _lib.lib
    N, K, group, M = 256, 1024, 128, 48
    rng, codes_h, s_h, z_h, bias_h = _layer(N, K, group, seed=7)
    codes = torch.from_numpy(codes_h).cuda()
    s, z = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in (s_h, z_h))
    x_h = orc.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    x = torch.from_numpy(x_h).cuda().to(torch.bfloat16)
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    out = {}

    def worker():
        out["rc"] = lib.lq_gemm_a16w4_fwd_static(_ptr(x), _ptr(codes), _ptr(s), _ptr(z), None, _ptr(got), M, N, K, group, None)
    t = threading.Thread(target=worker)
    t.start(); t.join()
    assert out["rc"] == 0, lib.lq_last_cuda_error()
    torch.cuda.synchronize()
    ref = orc.gemm_a16w4(x_h, codes_h, s_h, z_h, N, K, group=group)
    err = np.abs(got.float().cpu().numpy().astype(np.float64) - ref).max() / np.abs(ref).max()
    assert err <= RTOL


def test_static_scratch_rejects_shapes_beyond_its_size():
    from latentq_llm_b200 import _lib
    lib = _lib.lib
    # a plan that needs more partial-sum space than the built-in array: refused before any launch
    M, N, K = 2048, 256, 131072
    if lib.lq_gemm_workspace_bytes(_lib.GEMM_A16W4_FWD, M, N, K) <= 8 << 20:
        pytest.skip("plan for this shape fits the array on this device")
    fake = C.c_void_p(4096)
    rc = lib.lq_gemm_a16w4_fwd_static(fake, fake, fake, fake, None, fake, M, N, K, 128, None)
    assert rc == _lib.LQ_EWORKSPACE
    assert b"8 MiB" in lib.lq_last_cuda_error()
