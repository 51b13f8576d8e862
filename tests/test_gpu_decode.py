"""GPU parity of the decode-side kernels (residual add + RMSNorm, RoPE + KV store, single-query attention,
silu*up) against the CPU oracle.  Tolerance: one bf16 ulp (2^-8 relative) on at least 99.5 % of the elements and
2^-6 of the largest magnitude on all (reduction order and transcendental implementations differ)."""
import numpy as np
import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from latentq_llm_b200 import ops as _ops
    return _ops


def _close(got, want, frac=0.995):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want) / np.maximum(np.abs(want), 1e-6)
    assert (err <= 2.0 ** -8 + 1e-9).mean() >= frac, (err <= 2.0 ** -8).mean()
    assert np.abs(got - want).max() <= 2.0 ** -6 * np.abs(want).max()


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("hf", [True, False])
@pytest.mark.parametrize("M,K", [(1, 4096), (16, 4096), (3, 11008), (64, 2048)])
def test_add_rmsnorm(ops, M, K, hf):
    rng = np.random.default_rng(M * 7 + K)
    h = orc.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    d = orc.bf16_round(rng.standard_normal((M, K)).astype(np.float32) * 0.5)
    gamma = orc.bf16_round((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    for delta in (d, None):
        hd_ = _bf(h)
        y = ops.add_rmsnorm(hd_, None if delta is None else _bf(delta), _bf(gamma), 1e-5, hf_rounding=hf)
        want_h, want_y = orc.rmsnorm(h, gamma, 1e-5, delta=delta, hf_rounding=hf)
        assert np.array_equal(hd_.float().cpu().numpy(), want_h)            # the residual stream is exact
        _close(y.float().cpu().numpy(), want_y)


@pytest.mark.parametrize("hf", [True, False])
@pytest.mark.parametrize("B,Hq,Hkv,hd", [(1, 32, 32, 128), (4, 8, 2, 64)])
def test_rope_kv_store(ops, B, Hq, Hkv, hd, hf):
    rng = np.random.default_rng(B + Hq)
    max_len = 96
    qkv = orc.bf16_round(rng.standard_normal((B, (Hq + 2 * Hkv) * hd)).astype(np.float32))
    pos = rng.integers(0, max_len, B).astype(np.int64)
    inv_freq = (1.0 / (10000.0 ** (np.arange(0, hd, 2, dtype=np.float32) / hd))).astype(np.float32)
    kc = torch.zeros((B, Hkv, max_len, hd), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    t = _bf(qkv)
    ops.rope_kv_store(t, torch.from_numpy(pos).cuda(), torch.from_numpy(inv_freq).cuda(), kc, vc, Hq, Hkv, hd, hf_rounding=hf)
    got = t.float().cpu().numpy()
    q = qkv[:, :Hq * hd].reshape(B, Hq, hd)
    k = qkv[:, Hq * hd:(Hq + Hkv) * hd].reshape(B, Hkv, hd)
    v = qkv[:, (Hq + Hkv) * hd:].reshape(B, Hkv, hd)
    _close(got[:, :Hq * hd].reshape(B, Hq, hd), orc.rope_rotate_half(q, pos[:, None], inv_freq, hf_rounding=hf))
    assert np.array_equal(got[:, Hq * hd:], qkv[:, Hq * hd:])              # k and v columns of the row are left alone
    kr = orc.rope_rotate_half(k, pos[:, None], inv_freq, hf_rounding=hf)
    kcn, vcn = kc.float().cpu().numpy(), vc.float().cpu().numpy()
    for b in range(B):
        _close(kcn[b, :, pos[b]], kr[b])
        assert np.array_equal(vcn[b, :, pos[b]], v[b])
        mask = np.ones(max_len, bool); mask[pos[b]] = False
        assert not kcn[b][:, mask].any() and not vcn[b][:, mask].any()     # nothing else was written


@pytest.mark.parametrize("B,Hq,Hkv,hd,max_len", [(1, 32, 32, 128, 1024), (16, 32, 32, 128, 640), (3, 8, 2, 64, 200), (64, 8, 8, 128, 96)])
def test_decode_attention(ops, B, Hq, Hkv, hd, max_len):
    rng = np.random.default_rng(B * 3 + hd)
    qkv = orc.bf16_round(rng.standard_normal((B, (Hq + 2 * Hkv) * hd)).astype(np.float32))
    kc = orc.bf16_round(rng.standard_normal((B, Hkv, max_len, hd)).astype(np.float32))
    vc = orc.bf16_round(rng.standard_normal((B, Hkv, max_len, hd)).astype(np.float32))
    pos = rng.integers(0, max_len, B).astype(np.int64)
    pos[0] = max_len - 1
    if B > 1:
        pos[1] = 0
    for _ in range(2):          # twice: the ticket counters must have been left at zero
        out = ops.decode_attention(_bf(qkv), torch.from_numpy(pos).cuda(), _bf(kc), _bf(vc), Hq, Hkv, hd)
        want = orc.decode_attention(qkv[:, :Hq * hd].reshape(B, Hq, hd), kc, vc, pos, hd ** -0.5)
        got = out.float().cpu().numpy().reshape(B, Hq, hd)
        assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()


@pytest.mark.parametrize("hf", [True, False])
def test_silu_mul(ops, hf):
    rng = np.random.default_rng(5)
    gu = orc.bf16_round((rng.standard_normal((7, 2 * 11008)) * 2).astype(np.float32))
    got = ops.silu_mul(_bf(gu), hf_rounding=hf).float().cpu().numpy()
    _close(got, orc.silu_mul(gu, hf_rounding=hf))


@pytest.mark.parametrize("hf", [True, False])
@pytest.mark.parametrize("M,I,K", [(1, 1024, 4096), (2, 544, 4096), (8, 1024, 1024), (16, 288, 2048), (48, 512, 1024)])
def test_fused_gate_up_silu(ops, M, I, K, hf):
    """silu(x·Wgate^T) * (x·Wup^T) from the fused 2I-row weight: one launch at decode sizes (streaming kernel for one
    or two tokens, row-block kernel up to 16), GEMM + silu*up beyond; against the oracle's dequantize-matmul-silu chain
    within two bf16 ulps of the largest magnitude."""
    rng = np.random.default_rng(M + I)
    w = orc.bf16_round((rng.standard_normal((2 * I, K)) * 0.02).astype(np.float32))
    s, z = orc.find_qparams(w, 128, 15, False)
    s, z = orc.bf16_round(s), orc.bf16_round(z)
    codes, _, _ = orc.a16w4_requant(s, z, w=w, codec=orc.CODEC_NONE, math_bf16=True)
    x = orc.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    got = ops.gemm_a16w4_fwd_silu(_bf(x), torch.from_numpy(codes).cuda(), _bf(s), _bf(z), I, K, hf_rounding=hf).float().cpu().numpy()
    gu = orc.gemm_a16w4(x, codes, s, z, 2 * I, K)
    want = orc.silu_mul(gu, hf_rounding=hf)
    # (both projections are rounded to bf16 before silu and the product: an ulp in either moves the product by up to two)
    assert np.abs(got - want).max() <= 2.0 ** -6 * np.abs(want).max()
    # and exactly what the two separate launches give (same GEMM kernels, same rounding points)
    sep = ops.silu_mul(ops.gemm_a16w4_fwd(_bf(x), torch.from_numpy(codes).cuda(), _bf(s), _bf(z), None, 2 * I, K), hf_rounding=hf)
    if M <= 16:
        assert np.array_equal(got, sep.float().cpu().numpy())


@pytest.mark.parametrize("B,V,D", [(1, 32000, 4096), (16, 32000, 4096), (3, 1027, 256), (64, 50272, 2048), (2, 8, 8)])
def test_argmax_embed(ops, B, V, D):
    """The end of a greedy step in one launch: the first maximum per row (ties, rows of equal values, a NaN, rows that do
    not start on 16-byte boundaries), positions advanced by one, the winners' embedding rows copied."""
    g = torch.Generator(device="cuda").manual_seed(B + V)
    logits = torch.randn(B, V, device="cuda", generator=g).to(torch.bfloat16)
    logits[0, V // 3] = logits[0].max()                  # a tie in the first row: the lower index wins
    logits[0, V - 1] = logits[0].max()
    if B > 1:
        logits[1] = 0.5                                  # all equal: index 0
    if B > 2:
        logits[2, V // 2] = float("nan")                 # NaN counts as the maximum
        logits[2, V // 2 + 3] = float("nan")
    embed = torch.randn(V, D, device="cuda", generator=g).to(torch.bfloat16)
    tok = torch.full((B,), -1, dtype=torch.long, device="cuda")
    pos = torch.arange(B, dtype=torch.long, device="cuda") + 5
    h = torch.zeros(B, D, dtype=torch.bfloat16, device="cuda")
    ops.argmax_embed(logits, tok, pos, embed, h)
    want = logits.float().argmax(-1)
    assert torch.equal(tok, want)
    assert torch.equal(pos, torch.arange(B, device="cuda") + 6)
    assert torch.equal(h, embed[want])
    # argmax alone, on a column slice (row stride != V)
    tok2 = torch.full((B,), -1, dtype=torch.long, device="cuda")
    ops.argmax_embed(logits[:, : V - 1], tok2)
    assert torch.equal(tok2, logits[:, : V - 1].float().argmax(-1))
