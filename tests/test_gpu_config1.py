"""The reference's CPU-runnable configuration at full size: one OPT-1.3B fc1-shaped latent layer (8192 x 2048, int4
asymmetric, group 128, fp32 scale/zero, W ~ N(0, 0.02) in bf16), an update ~ N(0, 1e-4) folded in with the
stochastic-rounding requantize under seeded uniform noise, then the dequantized linear forward on [4*512, 2048]
activations.  Codes and residual words must equal the CPU oracle bit for bit; the forward within 1e-2 relative."""
import numpy as np
import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu


def test_config1_full_size():
    from latentq_llm_b200 import ops
    N, K, M = 8192, 2048, 2048
    g = torch.Generator().manual_seed(1234)
    w0 = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).float()
    delta = torch.randn(N, K, generator=g) * 1e-4
    noise = torch.empty(N * K).uniform_(-0.5, 0.5, generator=g)
    x = torch.randn(M, K, generator=g)
    # oracle (fp32 chain, the reference's CPU arithmetic)
    s, z = orc.find_qparams(w0.numpy(), 128, 15, False)
    c0, _, _ = orc.a16w4_requant(s, z, w=w0.numpy(), codec=orc.CODEC_NONE)
    c1, w1, _ = orc.a16w4_requant(s, z, codes=c0, delta=delta.numpy(), codec=orc.CODEC_UNIFORM16, dither=noise.numpy(),
                                  has_residual=False)
    # device
    sd, zd = ops.find_qparams(w0.cuda(), 128, 15, False)
    assert np.array_equal(sd.cpu().numpy(), s) and np.array_equal(zd.cpu().numpy(), z)
    codes, _ = ops.a16w4_requant(w0.cuda(), sd, zd, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.float32))
    assert np.array_equal(codes.cpu().numpy(), c0)
    words = torch.zeros(N * K // 8, dtype=torch.int32, device="cuda")
    o = ops.make_opts(codec=ops.CODEC_UNIFORM16, dither=ops.DITHER_EXPLICIT, math_dtype=torch.float32, res_round_bf16=False,
                      has_residual=False, dither_buf=noise.cuda())
    ops.a16w4_fold_delta(codes, words, delta.cuda().reshape(-1), sd, zd, o)
    assert np.array_equal(codes.cpu().numpy(), c1)
    assert np.array_equal(words.cpu().numpy(), w1)
    carries = int((np.unpackbits(np.frombuffer(c1.tobytes(), np.uint8)).sum()))      # just a checksum of the codes
    assert carries > 0
    # dequantized linear forward: fp32 on CPU (reference) vs the bf16 tensor-core kernel
    W = torch.from_numpy(orc.a16w4_dequant(c1, s, z)).view(N, K)
    y_ref = x.mm(W.t())
    y = ops.gemm_a16w4_fwd(x.cuda().to(torch.bfloat16), codes, sd.to(torch.bfloat16), zd.to(torch.bfloat16), None, N, K)
    err = (y.float().cpu() - y_ref).abs().max() / y_ref.abs().max()
    fro = (y.float().cpu() - y_ref).norm() / y_ref.norm()
    assert float(err) < 1e-2 and float(fro) < 1e-2, (float(err), float(fro))
