"""The oracle's decode-side operations against the eager modules the reference's fused kernels replace
(LlamaRMSNorm, apply_rotary_pos_emb, LlamaMLP's activation, scaled_dot_product_attention), on the CPU in bf16.
Transcendentals and reduction order differ between implementations, so the bar is one bf16 ulp (2^-8 relative)
on almost every element and 2^-6 on all."""
import numpy as np
import torch

import oracle as orc


def _close(got, want, frac=0.995):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want) / np.maximum(np.abs(want), 1e-6)
    assert (err <= 2.0 ** -8 + 1e-9).mean() >= frac, (err <= 2.0 ** -8).mean()
    assert np.abs(got - want).max() <= 2.0 ** -6 * np.abs(want).max()


def _bf(t):
    return t.to(torch.bfloat16)


def test_rmsnorm_matches_llama_rmsnorm():
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    g = torch.Generator().manual_seed(0)
    M, K = 5, 512
    norm = LlamaRMSNorm(K, eps=1e-5).to(torch.bfloat16)
    norm.weight.data = _bf(1.0 + 0.1 * torch.randn(K, generator=g))
    h, d = _bf(torch.randn(M, K, generator=g)), _bf(torch.randn(M, K, generator=g))
    want_h = h + d
    want_y = norm(want_h)
    got_h, got_y = orc.rmsnorm(h.float().numpy(), norm.weight.float().detach().numpy(), 1e-5, delta=d.float().numpy())
    assert np.array_equal(got_h, want_h.float().numpy())
    _close(got_y, want_y.float().detach().numpy())


def test_rope_matches_apply_rotary_pos_emb():
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    g = torch.Generator().manual_seed(1)
    B, H, hd = 3, 4, 128
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    pos = torch.tensor([0, 17, 733])
    q, k = _bf(torch.randn(B, H, 1, hd, generator=g)), _bf(torch.randn(B, H, 1, hd, generator=g))
    freqs = pos[:, None].float() * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], -1)
    cos, sin = _bf(emb.cos())[:, None, :], _bf(emb.sin())[:, None, :]          # [B, 1(seq), hd]
    wq, wk = apply_rotary_pos_emb(q, k, cos, sin)
    gq = orc.rope_rotate_half(q[:, :, 0].float().numpy(), pos.numpy()[:, None], inv_freq.numpy())
    gk = orc.rope_rotate_half(k[:, :, 0].float().numpy(), pos.numpy()[:, None], inv_freq.numpy())
    _close(gq, wq[:, :, 0].float().numpy())
    _close(gk, wk[:, :, 0].float().numpy())


def test_silu_mul_matches_llama_mlp_activation():
    g = torch.Generator().manual_seed(2)
    M, I = 4, 256
    gu = _bf(torch.randn(M, 2 * I, generator=g) * 2)
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    _close(orc.silu_mul(gu.float().numpy()), want.float().numpy())


def test_decode_attention_matches_sdpa():
    g = torch.Generator().manual_seed(3)
    B, Hq, Hkv, hd, L = 2, 8, 4, 64, 40
    q = _bf(torch.randn(B, Hq, 1, hd, generator=g))
    kc, vc = _bf(torch.randn(B, Hkv, L, hd, generator=g)), _bf(torch.randn(B, Hkv, L, hd, generator=g))
    pos = [11, 39]
    got = orc.decode_attention(q[:, :, 0].float().numpy(), kc.float().numpy(), vc.float().numpy(), pos, hd ** -0.5)
    for b in range(B):
        n = pos[b] + 1
        kk = kc[b:b + 1, :, :n].repeat_interleave(Hq // Hkv, dim=1).float()
        vv = vc[b:b + 1, :, :n].repeat_interleave(Hq // Hkv, dim=1).float()
        want = torch.nn.functional.scaled_dot_product_attention(q[b:b + 1].float(), kk, vv)
        assert np.abs(got[b] - want[0, :, 0].numpy()).max() <= 2.0 ** -7 * np.abs(want.numpy()).max()
