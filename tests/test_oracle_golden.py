"""The CPU oracle against vectors produced by executing the reference's own functions
(tests/golden/gen_golden.py).  Integer results must match bit for bit; fp32 results too,
since the oracle restates the same separately-rounded fp32 operations."""
import numpy as np

import oracle as orc


def test_pack_unpack(golden):
    assert np.array_equal(orc.pack_nibbles(golden["pack_codes"]), golden["pack_packed"])
    assert np.array_equal(orc.unpack_nibbles(golden["pack_packed"]), golden["unpack_codes"])
    assert np.array_equal(orc.unpack_nibbles(golden["pack_packed"]).astype(np.uint8), golden["pack_codes"])


def test_find_qparams(golden):
    for sym in (0, 1):
        s, z = orc.find_qparams(golden["qp_w"], 128, 15, bool(sym))
        assert np.array_equal(s, golden[f"qp_scale_sym{sym}"])
        assert np.array_equal(z, golden[f"qp_zero_sym{sym}"])


def _qp(golden):
    return golden["qp_scale_sym0"], golden["qp_zero_sym0"]


def test_requant_no_codec_fp32_and_bf16(golden):
    s, z = _qp(golden)
    codes, words, _ = orc.a16w4_requant(s, z, w=golden["qp_w"], codec=orc.CODEC_NONE)
    assert words is None and np.array_equal(codes, golden["rq_none_codes_f32"])
    sb, zb = orc.bf16_round(s), orc.bf16_round(z)
    codes, _, _ = orc.a16w4_requant(sb, zb, w=golden["rq_none_w_bf16"], codec=orc.CODEC_NONE, math_bf16=True)
    assert np.array_equal(codes, golden["rq_none_codes_bf16"])


def test_dequant(golden):
    s, z = _qp(golden)
    assert np.array_equal(orc.a16w4_dequant(golden["rq_none_codes_f32"], s, z), golden["dq_f32"].ravel())
    sb, zb = orc.bf16_round(s), orc.bf16_round(z)
    got = orc.a16w4_dequant(golden["rq_none_codes_f32"], sb, zb, math_bf16=True, out_bf16=True)
    assert np.array_equal(got, golden["dq_bf16"].ravel())


def test_uniform16_codec(golden):
    words, carry = orc.uniform16_encode(golden["u16_r"], golden["u16_noise"])
    assert np.array_equal(words, golden["u16_words"])
    assert np.array_equal(carry, golden["u16_carry"])
    assert carry.sum() > 0
    assert np.array_equal(orc.uniform16_decode(words), golden["u16_decode"])


def test_config1_two_steps(golden):
    s, z = _qp(golden)
    c1, w1, _ = orc.a16w4_requant(s, z, codes=golden["c1_codes0"], words=None, delta=golden["c1_delta"],
                                  codec=orc.CODEC_UNIFORM16, dither=golden["c1_noise1"], has_residual=False)
    assert np.array_equal(c1, golden["c1_codes1"])
    assert np.array_equal(w1, golden["c1_words1"])
    c2, w2, _ = orc.a16w4_requant(s, z, codes=c1, words=w1, delta=golden["c1_delta2"],
                                  codec=orc.CODEC_UNIFORM16, dither=golden["c1_noise2"], has_residual=True)
    assert np.array_equal(c2, golden["c1_codes2"])
    assert np.array_equal(w2, golden["c1_words2"])
    W = orc.a16w4_dequant(c2, s, z).reshape(64, 256)
    y = golden["c1_x"].astype(np.float64) @ W.astype(np.float64).T
    assert np.allclose(y, golden["c1_y"], rtol=1e-4, atol=1e-5)


def test_a8w8_requant(golden):
    c, w, _ = orc.a8w8_requant(golden["a8_qscales"], 32, 128, w=golden["a8_w"], codec=orc.CODEC_UNIFORM16,
                               dither=golden["a8_noise"])
    assert np.array_equal(c, golden["a8_codes"].ravel())
    assert np.array_equal(w, golden["a8_words"])
    c, _, _ = orc.a8w8_requant(golden["a8_qscales"], 32, 128, w=golden["a8_w"], codec=orc.CODEC_NONE)
    assert np.array_equal(c, golden["a8_codes_none"].ravel())


def test_opt8_codec(golden):
    q, s, t = orc.opt8_quant(golden["o8_x"], 2048)
    assert np.array_equal(q, golden["o8_q"])
    assert np.array_equal(s, golden["o8_scale"]) and np.array_equal(t, golden["o8_tmax"])
    assert np.array_equal(orc.opt8_dequant(q, 2048, s, t), golden["o8_deq"])


def test_act_quant_per_token(golden):
    q, s = orc.act_quant_per_token(golden["aq_x"])
    assert np.array_equal(q.astype(np.float32) * s[:, None], golden["aq_fake"])


def test_philox_known_answers():
    # Known-answer vectors of Philox4x32-10 from the Random123 distribution (kat_vectors).
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        assert tuple(int(v) for v in orc.philox4x32_10(ctr, key)) == want
    d = orc.philox_dither(1234, 7, 64)
    assert d.min() >= -0.5 and d.max() < 0.5 and abs(d.mean()) < 0.1


# ---- CUDA residual codecs: fixtures produced by the reference's own kernel text compiled for the CPU
# (oracle/build_ref.py; the bf16 inputs are the codec's WHOLE input domain, every bf16 value with |x| <= 0.5) ----
def _flags(x):
    return np.packbits(x != 0)


def test_threefold_codec_pinned_by_reference_kernels(golden):
    _, xb = orc.bf16_codec_domain()
    for mu in range(4):
        w, fl = orc.res3_quant(xb, mu)
        assert np.array_equal(w, golden[f"rc_q_bf16_words_mu{mu}"])
        assert np.array_equal(_flags(fl), golden[f"rc_q_bf16_flags_mu{mu}"])
        w, fl = orc.res3_quant(orc.f32_codec_grid(mu), mu)
        assert np.array_equal(w, golden[f"rc_q_f32_words_mu{mu}"])
        assert np.array_equal(_flags(fl), golden[f"rc_q_f32_flags_mu{mu}"])
        nib = golden["rc_all_nibbles"]
        assert np.array_equal(orc.res3_dequant(nib, mu, out_bf16=True), golden[f"rc_dq_bf16_mu{mu}"])
        assert np.array_equal(orc.res3_dequant(nib, mu, out_bf16=False), golden[f"rc_dq_f32_mu{mu}"])
        # launcher constants (.cu:346-351, 385-389): c1 c2 c3 | ic1 ic2 ic3 | b1 b2 t1 t2
        c = orc.curve_constants(*orc.curve_args(mu))
        assert np.array_equal(c[[0, 1, 2, 6, 7, 8, 9]], golden[f"rc_q_consts_mu{mu}"][:7])
        assert golden[f"rc_q_consts_mu{mu}"][7] == 0.0          # v0 = rand()%1000/1000 is integer division: always 0
        assert np.array_equal(c[[3, 4, 5, 6, 7, 8, 9]], golden[f"rc_dq_consts_mu{mu}"])
    assert golden["rc_q_bf16_flags_mu0"].any() and golden["rc_q_f32_flags_mu3"].any()   # carries do occur


def test_uniform_ext_codecs_pinned_by_reference_kernels(golden):
    _, xb = orc.bf16_codec_domain()
    w, fl = orc.resu_quant(xb)
    assert np.array_equal(w, golden["rc_uq_bf16_words"]) and np.array_equal(_flags(fl), golden["rc_uq_bf16_flags"])
    xg = orc.f32_codec_grid(0, seed=77)
    w, fl = orc.resu_quant(xg)
    assert np.array_equal(w, golden["rc_uq_f32_words"]) and np.array_equal(_flags(fl), golden["rc_uq_f32_flags"])
    w, fl = orc.resu_quant_s(xg)
    assert np.array_equal(w, golden["rc_uqs_f32_words"]) and np.array_equal(_flags(fl), golden["rc_uqs_f32_flags"])
    assert np.array_equal(orc.resu_dequant(golden["rc_all_nibbles"]), golden["rc_udq_f32"])
    assert np.array_equal(orc.resu_dequant(golden["rc_all_nibbles"]), golden["rc_udq_bf16"])


def test_reference_kernels_fma_contraction_is_immaterial(golden):
    # The reference's kernel text was compiled with and without contraction of a*b+c; both builds produced the same
    # bytes for every fixture above, so the restatement's fmaf() reading (nvcc's default) is not a guess there.
    assert bool(golden["rc_variants_agree"][0])


def test_reference_kernels_direct_when_built():
    # With oracle/_ref present (a container that holds the reference checkout), compare on a larger random sample.
    import ctypes as C
    libs = [orc.ref_codec(v) for v in ("fma", "nofma")]
    if any(L is None for L in libs):
        import pytest
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    rng = np.random.default_rng(99)
    for mu in range(4):
        k1, b1, k2, b2, k3 = orc.curve_args(mu)
        x = rng.uniform(-0.5, 0.5, 1 << 18).astype(np.float32)
        w, fl = orc.res3_quant(x, mu)
        for L in libs:
            xx = x.copy(); y = np.empty(x.size // 8, np.int32)
            L.ref_quant_f32(xx.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), k1, C.c_float(b1), k2,
                            C.c_float(b2), k3, y.size, None)
            assert np.array_equal(y, w) and np.array_equal(xx, fl)


# ---- a14: activation quantizer of QLinearFunctionA8W8_dynamic.forward (utils/quant.py:260-266) ----
def test_act_quant_per_tensor_golden(golden):
    for tag, bf in (("f32", False), ("bf16", True)):
        x = golden[f"pt_x_{tag}"]
        cv = float(golden[f"pt_clampv_{tag}"][0])
        assert cv == x.max()
        assert np.array_equal(orc.act_quant_per_tensor(x, cv, math_bf16=bf), golden[f"pt_x8_{tag}"])
        alpha = np.float32(cv) / np.float32(127.0)
        assert (orc.bf16_round(alpha) if bf else alpha) == golden[f"pt_alpha_{tag}"][0]


# ---- a18: three MyAdam.update_step steps as the reference executed them on the CPU ----
def test_adam_steps_golden(golden):
    g = golden
    n = g["adam_w"].size
    nb = n // 2048
    lat, s, z = g["adam_w"], g["adam_scales"], g["adam_zeros"]
    st1, st2 = np.zeros(n, np.uint8), np.zeros(n, np.uint8)          # init_state, utils/quant.py:1029-1059
    sc1, tm1 = np.full(nb, 1e-10, np.float32), np.zeros(nb, np.float32)
    sc2, tm2 = sc1.copy(), tm1.copy()
    for step in (1, 2, 3):
        codes, lat, st1, sc1, tm1, st2, sc2, tm2 = orc.adam_a16w4_step_cpu(
            lat, g[f"adam_grad{step - 1}"], s, z, st1, sc1, tm1, st2, sc2, tm2,
            beta1=0.9, beta2=0.95, eps=1e-8, lr=1e-3, step=step)
        assert np.array_equal(codes, g[f"adam_codes{step}"].ravel())
        assert np.array_equal(lat, g[f"adam_latent{step}"].ravel())
        assert np.array_equal(st1, g[f"adam_state1_{step}"].ravel())
        assert np.array_equal(st2, g[f"adam_state2_{step}"].ravel())
        for a, k in ((sc1, "qmap1"), (tm1, "absmax1"), (sc2, "qmap2"), (tm2, "absmax2")):
            assert np.array_equal(a, g[f"adam_{k}_{step}"])


# ---- GradientQTensor (utils/quant.py:846-921) as the reference's class executed it on the CPU ----
def test_gradient_accumulator_golden(golden):
    for tag, bf in (("f32", False), ("bf16", True)):
        q, sc = orc.gradq_accumulate(golden[f"gq_f0_{tag}"], golden[f"gq_noise0_{tag}"], math_bf16=bf)
        assert np.array_equal(q, golden[f"gq_q0_{tag}"]) and np.array_equal(sc, golden[f"gq_scale_{tag}"])
        for it in (1, 2):
            q, sc = orc.gradq_accumulate(golden[f"gq_f{it}_{tag}"], golden[f"gq_noise{it}_{tag}"], qdata=q, scale=sc, math_bf16=bf)
            assert np.array_equal(q, golden[f"gq_q{it}_{tag}"])
        val = q.astype(np.float32) * sc[:, None]
        assert np.array_equal(orc.bf16_round(val) if bf else val, golden[f"gq_value_{tag}"])
