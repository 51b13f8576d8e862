"""The allocation-free forward GEMM (`lq_gemm_a16w4_fwd_static`) against the workspace variant.

Some users of this library cannot allocate device memory where they call it: they run under a
framework that owns the whole device heap, or in a serving loop where an allocation's device-wide
synchronisation is not acceptable.  For them the split-K partial sums live in an array built into
the library.  This test drives the entry point through the C ABI exactly as such a caller would
(no workspace argument), twice in a row with different inputs, and compares each result with
`lq_gemm_a16w4_fwd` on the same inputs.  The second call also shows that whatever the first call
left in the shared array does not leak into a later result.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
RTOL = 1e-2   # the tolerance the other GEMM tests use; the two variants share their arithmetic


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def test_static_scratch_forward_matches_workspace_variant_twice():
    from latentq_llm_b200 import _lib, ops
    lib = _lib.lib
    N, K, group = 512, 1024, 128
    assert lib.lq_gemm_a16w4_fwd_static_max_bytes() == 8 << 20
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(2024)
    for call, M in enumerate((16, 5)):
        # this shape's plan really splits K, i.e. the built-in scratch is in use
        need = lib.lq_gemm_workspace_bytes(_lib.GEMM_A16W4_FWD, M, N, K)
        assert 0 < need <= 8 << 20
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        s, z = ops.find_qparams(w, group, 15, False)
        sb, zb = s.to(torch.bfloat16), z.to(torch.bfloat16)
        codes, _ = ops.a16w4_requant(w, sb, zb, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16), group=group)
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        want = ops.gemm_a16w4_fwd(x, codes, sb, zb, bias, N, K, group=group)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.lq_gemm_a16w4_fwd_static(_ptr(x), _ptr(codes), _ptr(sb), _ptr(zb), _ptr(bias), _ptr(got), M, N, K, group, stream)
        assert rc == 0, (call, rc, lib.lq_last_cuda_error())
        torch.cuda.synchronize()
        assert lib.lq_gemm_device_status(1) == 0
        assert not torch.isnan(got.float()).any()
        err = (got.double() - want.double()).abs().max() / want.double().abs().max()
        assert float(err) <= RTOL, (call, float(err))


def test_static_scratch_rejects_shapes_beyond_its_size():
    from latentq_llm_b200 import _lib
    lib = _lib.lib
    # a plan that would need more partial-sum space than the built-in array: refused before any launch
    M, N, K = 2048, 256, 131072
    if lib.lq_gemm_workspace_bytes(_lib.GEMM_A16W4_FWD, M, N, K) <= 8 << 20:
        pytest.skip("plan for this shape fits the array on this device")
    fake = C.c_void_p(4096)
    rc = lib.lq_gemm_a16w4_fwd_static(fake, fake, fake, fake, None, fake, M, N, K, 128, None)
    assert rc == _lib.LQ_EWORKSPACE
    assert b"8 MiB" in lib.lq_last_cuda_error()
