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
