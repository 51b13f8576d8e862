"""GPU parity of the streaming kernels against the CPU oracle (bit-exact) and the reference's golden vectors."""
import numpy as np
import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from latentq_llm_b200 import ops as _ops
    return _ops


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def test_pack_unpack_golden(ops, golden):
    packed = ops.pack_nibbles(dev(golden["pack_codes"]))
    assert np.array_equal(packed.cpu().numpy(), golden["pack_packed"])
    assert np.array_equal(ops.unpack_nibbles(packed).cpu().numpy(), golden["unpack_codes"])


def test_find_qparams_golden(ops, golden):
    for sym in (0, 1):
        s, z = ops.find_qparams(dev(golden["qp_w"]), 128, 15, bool(sym))
        assert np.array_equal(s.cpu().numpy(), golden[f"qp_scale_sym{sym}"])
        assert np.array_equal(z.cpu().numpy(), golden[f"qp_zero_sym{sym}"])
    # bf16 input, odd group size
    w = torch.randn(96 * 40, device="cuda").to(torch.bfloat16)
    s, z = ops.find_qparams(w, 96, 15, False)
    so, zo = orc.find_qparams(w.float().cpu().numpy(), 96, 15, False)
    assert np.array_equal(s.cpu().numpy(), so) and np.array_equal(z.cpu().numpy(), zo)


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("sym", [False, True])
def test_find_qparams_bf16_packed_kernel_vs_oracle(ops, group, sym):
    """The packed bf16 min/max kernel (groups of 32..256): ragged tail, an all-zero group, all-positive and all-negative
    groups (min and max are clamped to include 0), the golden weights rounded to bf16."""
    g = torch.Generator(device="cuda").manual_seed(group)
    n_groups = 4 * 1024 // group * 7 + 3                         # not a multiple of the 1024-element warp step
    w = (torch.randn(n_groups, group, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w[1] = 0
    w[2] = w[2].abs() + 0.01
    w[3] = -w[3].abs() - 0.01
    w[5, 0] = 3.0
    s, z = ops.find_qparams(w.reshape(-1), group, 15, sym)
    so, zo = orc.find_qparams(w.float().cpu().numpy(), group, 15, sym)
    assert np.array_equal(s.cpu().numpy(), so) and np.array_equal(z.cpu().numpy(), zo)


def test_dequant_golden(ops, golden):
    s, z = golden["qp_scale_sym0"], golden["qp_zero_sym0"]
    codes = dev(golden["rq_none_codes_f32"])
    out = ops.a16w4_dequant(codes, dev(s), dev(z), (64, 256), torch.float32)
    assert np.array_equal(out.cpu().numpy(), golden["dq_f32"])
    out = ops.a16w4_dequant(codes, dev(s, torch.bfloat16), dev(z, torch.bfloat16), (64, 256), torch.bfloat16)
    assert np.array_equal(out.float().cpu().numpy(), golden["dq_bf16"])


def test_uniform16_codec_golden(ops, golden):
    words, carry = ops.uniform16_encode(dev(golden["u16_r"]), dev(golden["u16_noise"]))
    assert np.array_equal(words.cpu().numpy(), golden["u16_words"])
    assert np.array_equal(carry.cpu().numpy(), golden["u16_carry"])
    assert np.array_equal(ops.uniform16_decode(words).cpu().numpy(), golden["u16_decode"])


def test_requant_golden_config1_steps(ops, golden):
    """Two optimizer steps of the CPU-reference configuration (fp32 chain, uniform codec, explicit noise)."""
    s, z = dev(golden["qp_scale_sym0"]), dev(golden["qp_zero_sym0"])
    o = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.float32)
    codes, _ = ops.a16w4_requant(dev(golden["qp_w"]), s, z, o)
    assert np.array_equal(codes.cpu().numpy(), golden["rq_none_codes_f32"])
    words = torch.zeros(codes.numel() // 4, dtype=torch.int32, device="cuda")
    o = ops.make_opts(codec=ops.CODEC_UNIFORM16, dither=ops.DITHER_EXPLICIT, math_dtype=torch.float32,
                      res_round_bf16=False, has_residual=False, dither_buf=dev(golden["c1_noise1"]))
    ops.a16w4_fold_delta(codes, words, dev(golden["c1_delta"]), s, z, o)
    assert np.array_equal(codes.cpu().numpy(), golden["c1_codes1"])
    assert np.array_equal(words.cpu().numpy(), golden["c1_words1"])
    o = ops.make_opts(codec=ops.CODEC_UNIFORM16, dither=ops.DITHER_EXPLICIT, math_dtype=torch.float32,
                      res_round_bf16=False, has_residual=True, dither_buf=dev(golden["c1_noise2"]))
    ops.a16w4_fold_delta(codes, words, dev(golden["c1_delta2"]), s, z, o)
    assert np.array_equal(codes.cpu().numpy(), golden["c1_codes2"])
    assert np.array_equal(words.cpu().numpy(), golden["c1_words2"])


def test_requant_bf16_chain_golden(ops, golden):
    s = dev(golden["qp_scale_sym0"], torch.bfloat16)
    z = dev(golden["qp_zero_sym0"], torch.bfloat16)
    o = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16)
    codes, _ = ops.a16w4_requant(dev(golden["rq_none_w_bf16"], torch.bfloat16), s, z, o)
    assert np.array_equal(codes.cpu().numpy(), golden["rq_none_codes_bf16"])


def test_a8w8_requant_golden(ops, golden):
    qs = dev(golden["a8_qscales"])
    o = ops.make_opts(codec=ops.CODEC_UNIFORM16, dither=ops.DITHER_EXPLICIT, math_dtype=torch.float32,
                      res_round_bf16=False, dither_buf=dev(golden["a8_noise"]))
    c, w = ops.a8w8_requant(dev(golden["a8_w"]), qs, o)
    assert np.array_equal(c.cpu().numpy(), golden["a8_codes"])
    assert np.array_equal(w.cpu().numpy(), golden["a8_words"])
    o = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.float32)
    c, _ = ops.a8w8_requant(dev(golden["a8_w"]), qs, o)
    assert np.array_equal(c.cpu().numpy(), golden["a8_codes_none"])


def test_opt8_golden(ops, golden):
    q, s, t = ops.opt8_quant(dev(golden["o8_x"]), 2048)
    assert np.array_equal(q.cpu().numpy(), golden["o8_q"])
    assert np.array_equal(s.cpu().numpy().ravel(), golden["o8_scale"])
    assert np.array_equal(t.cpu().numpy().ravel(), golden["o8_tmax"])
    assert np.array_equal(ops.opt8_dequant(q, 2048, s, t).cpu().numpy(), golden["o8_deq"])
    x = np.random.default_rng(3).standard_normal(128 * 9).astype(np.float32)
    q, s, t = ops.opt8_quant(dev(x), 128)
    qo, so, to = orc.opt8_quant(x, 128)
    assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy().ravel(), so)


def _edge_residuals(n, rng):
    r = (rng.random(n, dtype=np.float32) - 0.5).astype(np.float32)
    r[:12] = [-0.5, 0.5, 0.0, 0.125, 0.25, -0.125, -0.25, 0.49, -0.49, 0.2666, 0.375, 0.4375]
    return r


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mu", [0, 1, 2, 3])
def test_threefold_codec_vs_oracle(ops, dtype, mu):
    rng = np.random.default_rng(10 + mu)
    r = _edge_residuals(8 * 4096, rng)
    x = dev(r, dtype)
    r_in = x.float().cpu().numpy()
    words = torch.empty(4096, dtype=torch.int32, device="cuda")
    k = orc.curve_args(mu)
    ops.res3_quant(x, words, *k)
    wo, fo = orc.res3_quant(r_in, mu)
    assert np.array_equal(words.cpu().numpy(), wo)
    assert np.array_equal(x.float().cpu().numpy(), fo)
    out = torch.empty(8 * 4096, dtype=dtype, device="cuda")
    ops.res3_dequant(words, out, *k)
    assert np.array_equal(out.float().cpu().numpy(), orc.res3_dequant(wo, mu, out_bf16=(dtype == torch.bfloat16)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_uniform_ext_codecs_vs_oracle(ops, dtype):
    rng = np.random.default_rng(5)
    x0 = dev(_edge_residuals(8 * 1024, rng), dtype)
    r_in = x0.float().cpu().numpy()
    words = torch.empty(1024, dtype=torch.int32, device="cuda")
    x = x0.clone(); ops.resu_quant(x, words)
    wo, fo = orc.resu_quant(r_in)
    assert np.array_equal(words.cpu().numpy(), wo) and np.array_equal(x.float().cpu().numpy(), fo)
    x = x0.clone(); ops.resu_quant_s(x, words)
    wo, fo = orc.resu_quant_s(r_in)
    assert np.array_equal(words.cpu().numpy(), wo) and np.array_equal(x.float().cpu().numpy(), fo)
    out = torch.empty(8 * 1024, dtype=dtype, device="cuda")
    ops.resu_dequant(words, out)
    assert np.array_equal(out.float().cpu().numpy(), orc.resu_dequant(wo))


@pytest.mark.parametrize("mu", [0, 1, 2, 3])
def test_threefold_codec_golden_reference_kernels(ops, golden, mu):
    """lq_res3_quant / lq_res3_dequant against what the reference's own kernel text computes (fixtures made by
    oracle/build_ref.py): every bf16 input of the codec's domain, and an fp32 grid with the segment boundaries."""
    k = orc.curve_args(mu)
    pats, _ = orc.bf16_codec_domain()
    for tag, x in (("bf16", torch.from_numpy(pats.view(np.int16)).cuda().view(torch.bfloat16)),
                   ("f32", dev(orc.f32_codec_grid(mu)))):
        words = torch.empty(x.numel() // 8, dtype=torch.int32, device="cuda")
        ops.res3_quant(x, words, *k)
        assert np.array_equal(words.cpu().numpy(), golden[f"rc_q_{tag}_words_mu{mu}"])
        assert np.array_equal(np.packbits(x.float().cpu().numpy() != 0), golden[f"rc_q_{tag}_flags_mu{mu}"])
    nib = dev(golden["rc_all_nibbles"])
    for tag, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        out = torch.empty(16, dtype=dt, device="cuda")
        ops.res3_dequant(nib, out, *k)
        assert np.array_equal(out.float().cpu().numpy(), golden[f"rc_dq_{tag}_mu{mu}"])


def test_uniform_ext_codecs_golden_reference_kernels(ops, golden):
    pats, _ = orc.bf16_codec_domain()
    x = torch.from_numpy(pats.view(np.int16)).cuda().view(torch.bfloat16)
    words = torch.empty(x.numel() // 8, dtype=torch.int32, device="cuda")
    ops.resu_quant(x, words)
    assert np.array_equal(words.cpu().numpy(), golden["rc_uq_bf16_words"])
    assert np.array_equal(np.packbits(x.float().cpu().numpy() != 0), golden["rc_uq_bf16_flags"])
    for fn, tag in ((ops.resu_quant, "uq"), (ops.resu_quant_s, "uqs")):
        x = dev(orc.f32_codec_grid(0, seed=77))
        words = torch.empty(x.numel() // 8, dtype=torch.int32, device="cuda")
        fn(x, words)
        assert np.array_equal(words.cpu().numpy(), golden[f"rc_{tag}_f32_words"])
        assert np.array_equal(np.packbits(x.cpu().numpy() != 0), golden[f"rc_{tag}_f32_flags"])
    nib = dev(golden["rc_all_nibbles"])
    for tag, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        out = torch.empty(16, dtype=dt, device="cuda")
        ops.resu_dequant(nib, out)
        assert np.array_equal(out.float().cpu().numpy(), golden[f"rc_udq_{tag}"])


def test_act_quant_per_tensor_golden(ops, golden):
    """The quantizer inside QLinearFunctionA8W8_dynamic.forward as the reference executed it on bf16 activations."""
    xb = dev(golden["pt_x_bf16"], torch.bfloat16)
    x8, clampv = ops.act_quant_per_tensor(xb)
    assert float(clampv) == float(golden["pt_clampv_bf16"][0])
    assert np.array_equal(x8.cpu().numpy(), golden["pt_x8_bf16"])


def test_philox_stream_matches_oracle(ops):
    d = ops.philox_dither(0x1234567887654321, (7 << 32) | 3, 4096, "cuda", first_word=(1 << 33) + 5)
    assert np.array_equal(d.cpu().numpy(), orc.philox_dither(0x1234567887654321, (7 << 32) | 3, 4096, first_word=(1 << 33) + 5))


def _layer(rng, N, K, group=128):
    w = orc.bf16_round((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    s, z = orc.find_qparams(w, group, 15, False)
    return w, s, z


@pytest.mark.parametrize("math", ["f32", "bf16"])
@pytest.mark.parametrize("codec,dither", [("u16", "explicit"), ("u16", "philox"), ("3f", "hash"), ("3f", "philox"),
                                          ("3f", "explicit")])
def test_fold_delta_vs_oracle(ops, math, codec, dither):
    """Three consecutive steps; codes and residual words must equal the oracle's bit for bit."""
    rng = np.random.default_rng(42)
    N, K = 96, 512
    bf = math == "bf16"
    w, s, z = _layer(rng, N, K)
    if bf:
        s, z = orc.bf16_round(s), orc.bf16_round(z)
    qdt = torch.bfloat16 if bf else torch.float32
    sd, zd = dev(s, qdt), dev(z, qdt)
    codec_id = orc.CODEC_UNIFORM16 if codec == "u16" else orc.CODEC_THREEFOLD
    dith_id = {"hash": ops.DITHER_HASH, "explicit": ops.DITHER_EXPLICIT, "philox": ops.DITHER_PHILOX}[dither]
    codes_o, _, _ = orc.a16w4_requant(s, z, w=w, codec=orc.CODEC_NONE, math_bf16=bf)
    codes_d = dev(codes_o)
    words_o, words_d = None, torch.zeros(N * K // 8, dtype=torch.int32, device="cuda")
    seed = 99
    for step in range(3):
        delta = (rng.standard_normal(N * K) * (2e-3 if step == 1 else 2e-4)).astype(np.float32)
        if bf:
            delta = orc.bf16_round(delta)
        mu_enc, mu_dec = (step % 4, (step - 1) % 4) if codec == "3f" else (0, 0)
        if dither == "explicit":
            dith = (rng.random(N * K, dtype=np.float32) - 0.5).astype(np.float32)
        elif dither == "philox":
            dith = orc.philox_dither(seed, (step << 32) | 5, N * K // 8)
        else:
            dith = None
        codes_o, words_o, _ = orc.a16w4_requant(s, z, codes=codes_o, words=words_o, delta=delta, codec=codec_id,
                                                math_bf16=bf, res_round_bf16=bf, has_residual=step > 0,
                                                mu_enc=mu_enc, mu_dec=mu_dec, dither=dith)
        o = ops.make_opts(codec=codec_id, dither=dith_id, math_dtype=qdt, res_round_bf16=bf, has_residual=step > 0,
                          mu_enc=mu_enc, mu_dec=mu_dec, seed=seed, step=step, param_id=5,
                          dither_buf=dev(dith) if dither == "explicit" else None)
        ops.a16w4_fold_delta(codes_d, words_d, dev(delta, qdt), sd, zd, o)
        assert np.array_equal(codes_d.cpu().numpy(), codes_o), f"codes differ at step {step}"
        assert np.array_equal(words_d.cpu().numpy(), words_o), f"residual words differ at step {step}"
    assert len(np.unique(codes_o)) > 16


@pytest.mark.parametrize("math", ["f32", "bf16"])
def test_a8w8_fold_delta_vs_oracle(ops, math):
    rng = np.random.default_rng(7)
    N, K = 64, 384
    bf = math == "bf16"
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    qs = (np.abs(w).max(axis=1) / 127.0).astype(np.float32)
    if bf:
        qs, w = orc.bf16_round(qs), orc.bf16_round(w)
    qdt = torch.bfloat16 if bf else torch.float32
    codes_o, words_o, _ = orc.a8w8_requant(qs, N, K, w=w, codec=orc.CODEC_THREEFOLD, math_bf16=bf, res_round_bf16=bf)
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=qdt, res_round_bf16=bf)
    codes_d, words_d = ops.a8w8_requant(dev(w, qdt), dev(qs, qdt), o)
    assert np.array_equal(codes_d.cpu().numpy().ravel(), codes_o) and np.array_equal(words_d.cpu().numpy(), words_o)
    for step in range(2):
        delta = (rng.standard_normal(N * K) * 3e-4).astype(np.float32)
        if bf:
            delta = orc.bf16_round(delta)
        codes_o, words_o, _ = orc.a8w8_requant(qs, N, K, codes=codes_o, words=words_o, delta=delta,
                                               codec=orc.CODEC_THREEFOLD, math_bf16=bf, res_round_bf16=bf)
        ops.a8w8_fold_delta(codes_d, words_d, dev(delta, qdt), dev(qs, qdt), o)
        assert np.array_equal(codes_d.cpu().numpy().ravel(), codes_o)
        assert np.array_equal(words_d.cpu().numpy(), words_o)


def test_requant_roundtrip_property_full_size(ops):
    """At the benchmark's layer size: folding a zero update with no dither noise reproduces the codes, and replicas
    given the same seed produce identical codes and residuals."""
    N, K = 8192, 2048
    g = torch.Generator(device="cuda").manual_seed(1)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    s, z = ops.find_qparams(w, 128, 15, False)
    sb, zb = s.to(torch.bfloat16), z.to(torch.bfloat16)
    o0 = ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16)
    codes, _ = ops.a16w4_requant(w, sb, zb, o0)
    deq = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16)
    codes2, _ = ops.a16w4_requant(deq, sb, zb, o0)
    assert torch.equal(codes, codes2)
    delta = (torch.randn(N * K, device="cuda", generator=g) * 1e-4).to(torch.bfloat16)
    outs = []
    for _ in range(2):
        c, wd = codes.clone(), torch.zeros(N * K // 8, dtype=torch.int32, device="cuda")
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_PHILOX, has_residual=False, seed=11, step=1, param_id=2)
        ops.a16w4_fold_delta(c, wd, delta, sb, zb, o)
        outs.append((c, wd))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    # an update of 1e-4 is far below one code step (~8e-3): it lands in the residual words, not in the codes
    assert torch.unique(outs[0][1]).numel() > 1000


@pytest.mark.parametrize("K", [2048, 4096, 8192, 11008])
def test_act_quant_per_token_row_sizes(ops, K):
    """Rows kept in registers (K <= 8192) and the re-reading variant (K > 8192), with outlier channels and a zero row."""
    rng = np.random.default_rng(K)
    x = rng.standard_normal((37, K)).astype(np.float32)
    x[:, ::97] *= 20.0
    x[5] = 0.0
    xb = dev(x, torch.bfloat16)
    x8, s = ops.act_quant_per_token(xb)
    qo, so = orc.act_quant_per_token(xb.float().cpu().numpy(), math_bf16=True)
    assert np.array_equal(x8.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy().ravel(), so.ravel())


def test_act_quant_vs_oracle(ops, golden):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((24, 512)).astype(np.float32)
    x[:, 3] *= 20.0
    xb = dev(x, torch.bfloat16)
    x8, s = ops.act_quant_per_token(xb)
    qo, so = orc.act_quant_per_token(xb.float().cpu().numpy(), math_bf16=True)
    assert np.array_equal(x8.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy(), so)
    x8, clampv = ops.act_quant_per_tensor(xb)
    cv = float(xb.float().max())
    assert float(clampv) == cv
    assert np.array_equal(x8.cpu().numpy(), orc.act_quant_per_tensor(xb.float().cpu().numpy(), cv, math_bf16=True))


def test_empty_and_bad_inputs(ops):
    e = torch.empty(0, dtype=torch.uint8, device="cuda")
    assert ops.pack_nibbles(e).numel() == 0
    from latentq_llm_b200._lib import LatentQError
    with pytest.raises(LatentQError):
        ops.find_qparams(torch.zeros(100, device="cuda"), 128)


@pytest.mark.parametrize("dither", ["hash", "philox"])
def test_fast_fold_path_equals_generic_kernel(ops, monkeypatch, dither):
    """The packed-bf16 / table-driven fast paths (hash dither: the reference's production configuration; Philox
    dither: threshold table) against the generic kernel on 4M weights, including weights far outside the quantization
    range (which the fast path hands to the generic code) and every pair of curve levels."""
    DITH = ops.DITHER_HASH if dither == "hash" else ops.DITHER_PHILOX
    N, K = 2048, 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    s, z = ops.find_qparams(w, 128, 15, False)
    sb, zb = s.to(torch.bfloat16), z.to(torch.bfloat16)
    codes0, _ = ops.a16w4_requant(w, sb, zb, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16))
    delta = (torch.randn(N * K, device="cuda", generator=g) * 2e-3).to(torch.bfloat16)
    delta[::4099] = 3.0          # |Z| far beyond 64 (hash table) / 32 (Philox table)
    delta[1::7919] = -0.7
    delta[2::10007] = float("inf")
    results = {}
    for mode in ("fast", "generic"):
        if mode == "generic":
            monkeypatch.setenv("LQ_REQUANT_GENERIC", "1")
        else:
            monkeypatch.delenv("LQ_REQUANT_GENERIC", raising=False)
        c, wd = codes0.clone(), torch.zeros(N * K // 8, dtype=torch.int32, device="cuda")
        outs = []
        for step, (mu_enc, mu_dec) in enumerate([(0, 0), (1, 0), (2, 1), (3, 2), (0, 3)]):
            o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=DITH, has_residual=step > 0, mu_enc=mu_enc, mu_dec=mu_dec,
                              seed=77, step=step, param_id=9)
            ops.a16w4_fold_delta(c, wd, delta if step != 3 else None, sb, zb, o)
            outs.append((c.clone(), wd.clone()))
        # requantize-from-latent entry as well
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=DITH, mu_enc=1, seed=77, step=9, param_id=9)
        outs.append(ops.a16w4_requant((w.float() + delta.view(N, K).float() * 0.1).to(torch.bfloat16), sb, zb, o))
        results[mode] = outs
    for (cf, wf), (cg, wg) in zip(results["fast"], results["generic"]):
        assert torch.equal(cf, cg) and torch.equal(wf, wg)
    # the fast path must really be the one that ran: only the words poisoned above may fall back to the generic code
    import ctypes
    from latentq_llm_b200 import _lib
    cnt = ctypes.c_ulonglong(0)
    monkeypatch.delenv("LQ_REQUANT_GENERIC", raising=False)
    _lib.lib.lq_fold_fallback_words(1, ctypes.byref(cnt))
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=DITH, has_residual=False, seed=1)
    c, wd = codes0.clone(), torch.zeros(N * K // 8, dtype=torch.int32, device="cuda")
    ops.a16w4_fold_delta(c, wd, delta, sb, zb, o)
    _lib.lib.lq_fold_fallback_words(1, ctypes.byref(cnt))
    poisoned = N * K // 4099 + N * K // 7919 + N * K // 10007 + 3
    assert 0 < cnt.value <= 2 * poisoned, (cnt.value, poisoned)     # a poisoned word takes its neighbour along


@pytest.mark.parametrize("N,K", [(1024, 4096), (517, 1736)])      # 512 and 217 (not a power of two) words per row
def test_fast_fold_path_int8_equals_generic_kernel(ops, monkeypatch, N, K):
    """A8W8 latent requantize: the table-driven bf16 fast path against the generic kernel, every variant (from dense
    weights, with / without residual, with / without update), weights beyond the int8 range and non-finite updates."""
    import ctypes
    from latentq_llm_b200 import _lib
    g = torch.Generator(device="cuda").manual_seed(6)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w[:, 5] *= 8.0
    qs = (w.float().abs().amax(dim=1) / 127.0).to(torch.bfloat16)
    delta = (torch.randn(N * K, device="cuda", generator=g) * 1e-4).to(torch.bfloat16)
    delta[::4099] = 3.0           # |Z| beyond 256: handed to the generic chain
    delta[1::7919] = float("-inf")
    delta[2::10007] = 0.05        # clamps at +127 inside the table
    results = {}
    cnt = ctypes.c_ulonglong(0)
    for mode in ("fast", "generic"):
        if mode == "generic":
            monkeypatch.setenv("LQ_REQUANT_GENERIC", "1")
        else:
            monkeypatch.delenv("LQ_REQUANT_GENERIC", raising=False)
        _lib.lib.lq_fold_fallback_words(1, ctypes.byref(cnt))
        outs = []
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=torch.bfloat16, mu_enc=1)
        c, wd = ops.a8w8_requant(w, qs, o)
        outs.append((c.clone(), wd.clone()))
        for step, (mu_enc, mu_dec) in enumerate([(0, 1), (1, 0), (2, 1), (3, 2), (0, 3)]):
            o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=torch.bfloat16,
                              has_residual=step != 1, mu_enc=mu_enc, mu_dec=mu_dec)
            ops.a8w8_fold_delta(c, wd, delta if step != 3 else None, qs, o)
            outs.append((c.clone(), wd.clone()))
        _lib.lib.lq_fold_fallback_words(1, ctypes.byref(cnt))
        if mode == "fast":
            poisoned = N * K // 4099 + N * K // 7919 + 2
            assert 0 < cnt.value <= 6 * poisoned, (cnt.value, poisoned)    # the fast kernel ran; only poisoned words left it
        results[mode] = outs
    for i, ((cf, wf), (cg, wg)) in enumerate(zip(results["fast"], results["generic"])):
        assert torch.equal(cf, cg), i
        assert torch.equal(wf, wg), i
    assert results["fast"][-1][0].unique().numel() > 100


def test_requant_beyond_2p32_elements(ops):
    """2^32 + 2^22 weights in one call (64-bit element indices, Philox counters beyond 2^29 words): slices at the start,
    across the 2^32-element boundary and at the very end equal the same slices requantized on their own (hash dither is
    position-independent), and the last words of the Philox run equal the oracle fed with the Philox stream at that
    word offset."""
    n = (1 << 32) + (1 << 22)
    g = torch.Generator(device="cuda").manual_seed(3)
    codes = torch.randint(-128, 128, (n // 2,), device="cuda", generator=g, dtype=torch.int8)
    words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n // 8,), device="cuda", generator=g, dtype=torch.int32)
    delta = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for a in range(0, n, 1 << 30):                                  # filled in pieces: no fp32 temporary of the full size
        b = min(n, a + (1 << 30))
        delta[a:b] = (torch.randn(b - a, device="cuda", generator=g, dtype=torch.float32) * 1e-3).to(torch.bfloat16)
    s = (0.004 + 0.004 * torch.rand(n // 128, device="cuda", generator=g)).to(torch.bfloat16)
    z = torch.randint(0, 16, (n // 128,), device="cuda", generator=g).to(torch.bfloat16)
    T = 1 << 20
    spans = [(0, T), ((1 << 32) - T // 2, (1 << 32) + T // 2), (n - T, n)]

    def cut(a, b):
        return (codes[a // 2:b // 2].clone(), words[a // 8:b // 8].clone(), delta[a:b].clone(),
                s[a // 128:b // 128].clone(), z[a // 128:b // 128].clone())

    # hash dither (the table-driven fast path)
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=torch.bfloat16, has_residual=True,
                      mu_enc=1, mu_dec=2)
    parts = [cut(a, b) for a, b in spans]
    ops.a16w4_fold_delta(codes, words, delta, s, z, o)
    for (a, b), (c, w, d, ss, zz) in zip(spans, parts):
        ops.a16w4_fold_delta(c, w, d, ss, zz, o)
        assert torch.equal(c, codes[a // 2:b // 2]) and torch.equal(w, words[a // 8:b // 8]), (a, b)
    # Philox dither: counters are 64-bit word indices
    nw = 4096
    a = n - 8 * nw
    c0, w0, d0, s0, z0 = cut(a, n)
    seed, stream = 0x1234567, (9 << 32) | 4
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_PHILOX, math_dtype=torch.bfloat16, has_residual=True,
                      mu_enc=2, mu_dec=1, seed=seed, step=9, param_id=4)
    assert o.stream_id == stream
    ops.a16w4_fold_delta(codes, words, delta, s, z, o)
    dith = orc.philox_dither(seed, stream, nw, first_word=n // 8 - nw)
    co, wo, _ = orc.a16w4_requant(s0.float().cpu().numpy(), z0.float().cpu().numpy(), codes=c0.cpu().numpy(),
                                  words=w0.cpu().numpy(), delta=d0.float().cpu().numpy(), codec=orc.CODEC_THREEFOLD,
                                  math_bf16=True, res_round_bf16=True, has_residual=True, mu_enc=2, mu_dec=1, dither=dith)
    assert np.array_equal(codes[a // 2:].cpu().numpy(), co) and np.array_equal(words[a // 8:].cpu().numpy(), wo)


@pytest.mark.parametrize("n", [2, 14, 16, 30, 4096 + 6, 1 << 20])
@pytest.mark.parametrize("offset", [0, 2])
def test_pack_unpack_vector_and_tail_paths(ops, n, offset):
    """16 codes per thread where the buffers are aligned, byte-wise for the tail and for unaligned views; codes beyond 15
    wrap like the reference's int8 arithmetic (python_compress, utils/quant.py:4-11: (a << 4) + b in int8)."""
    g = torch.Generator(device="cuda").manual_seed(n + offset)
    raw = torch.randint(0, 256, (n + offset,), device="cuda", generator=g, dtype=torch.uint8)
    codes = raw[offset:]
    packed = ops.pack_nibbles(codes)
    want = ((codes[0::2].to(torch.int32) << 4) + codes[1::2].to(torch.int32)) & 255
    assert torch.equal(packed.view(torch.uint8).to(torch.int32), want)
    small = codes & 15
    packed = ops.pack_nibbles(small)
    back = ops.unpack_nibbles(packed)
    assert torch.equal(back.view(torch.uint8), small)
    if offset:                                      # unpack from an unaligned packed view
        buf = torch.zeros(packed.numel() + offset, device="cuda", dtype=torch.int8)
        buf[offset:] = packed
        assert torch.equal(ops.unpack_nibbles(buf[offset:]).view(torch.uint8), small)
