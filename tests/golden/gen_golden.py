"""Generate the golden vectors under tests/golden/ by EXECUTING the reference's own code.

Run once in a container that has the reference checkout (it does not travel
to the GPU box; the .npz files do):

    python tests/golden/gen_golden.py /path/to/latentQ_LLM

`utils/quant.py` cannot be imported (it needs torch_int, a GPU and a JIT
build at import time), so the pure-torch functions are loaded by slicing the
module's AST: the selected `def`s / assignments are compiled from the
reference file where it lies and executed in a scratch namespace.  Nothing
from the reference is copied into this repository.

`ResidualTensor` allocates on 'cuda' in its constructor, so a CPU stand-in
with the same `set_value(residual_fp, scale) -> carry flags` contract is put in
the namespace; it routes to the reference's own CPU codec
(`python_quant_linear`, utils/quant.py:765-778), which is what the reference's
`cuda_quant_linear` does for CPU tensors (utils/quant.py:728-729).
"""
import ast
import os
import sys

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))


def slice_module(path, names, extra_ns=None):
    src = open(path).read()
    tree = ast.parse(src)
    keep = []
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in names:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in names for t in node.targets):
            keep.append(node)
    mod = ast.Module(body=keep, type_ignores=[])
    ns = {"torch": torch, "nn": torch.nn, "math": __import__("math"), "np": np}
    ns.update(extra_ns or {})
    exec(compile(mod, path, "exec"), ns)
    return ns


def f32(t):
    return t.detach().to(torch.float32).contiguous().numpy()


def main(ref):
    qpath = os.path.join(ref, "utils", "quant.py")

    class ResidualTensor:  # CPU stand-in, see module docstring
        def __init__(self):
            self.residual_int = None
            self.noise_seed = None

        def set_value(self, residual_fp, weight_scale=None):
            if self.noise_seed is not None:
                torch.manual_seed(self.noise_seed)
            words, adj = ns["python_quant_linear"](residual_fp.contiguous())
            self.residual_int = words
            return adj.view(residual_fp.shape)

    ns = slice_module(qpath, {"python_compress", "python_decompress", "Qfunc_8bit_opt", "DeQfunc_8bit_opt",
                              "GROUPSIZE", "Qfunc_4bit_g_res", "DeQfunc_4bit_g", "Qfunc_8bit_res",
                              "python_quant_linear", "python_dequant_linear", "three_fold_curve_4bit"},
                      {"ResidualTensor": ResidualTensor})
    qz = slice_module(os.path.join(ref, "PTQ", "quant", "quantizer.py"), {"Quantizer"})
    ql = slice_module(os.path.join(ref, "PTQ", "quant", "quant_linear.py"),
                      {"quantize_activation_per_token_absmax"})

    g = torch.Generator().manual_seed(1234)
    out = {}

    # --- a1/a2 pack / unpack ------------------------------------------------
    codes = torch.randint(0, 16, (4096,), generator=g, dtype=torch.uint8)
    codes[:32] = torch.arange(32, dtype=torch.uint8) % 16
    packed = ns["python_compress"](codes.clone())
    out["pack_codes"] = codes.numpy()
    out["pack_packed"] = packed.numpy()
    out["unpack_codes"] = ns["python_decompress"](packed).numpy().reshape(-1)

    # --- a19 group min/max ---------------------------------------------------
    W = (torch.randn(64, 256, generator=g) * 0.02).to(torch.bfloat16).float()
    W[3, :128] = 0.0                       # all-zero group -> (-1, +1) rule
    W[5, 128:] = W[5, 128:].abs()          # all-positive group -> xmin clamps to 0
    for sym in (False, True):
        q = qz["Quantizer"]()
        q.configure(4, perchannel=True, sym=sym, mse=False)
        q.find_params(W.view(-1, 128), weight=True)
        out[f"qp_scale_sym{int(sym)}"] = f32(q.scale.reshape(-1))
        out[f"qp_zero_sym{int(sym)}"] = f32(q.zero.reshape(-1))
    out["qp_w"] = f32(W)
    q = qz["Quantizer"]()
    q.configure(4, perchannel=True, sym=False, mse=False)
    q.find_params(W.view(-1, 128), weight=True)
    scales, zeros = q.scale.reshape(-1, 1).clone(), q.zero.reshape(-1, 1).clone()
    shape = [64, 256]

    # --- a6 without a residual codec (lbit=16 handle), fp32 and bf16 chains --
    class Plain:
        dtype = torch.float32
        data = None
    codes0 = ns["Qfunc_4bit_g_res"](W.clone(), Plain(), [scales, zeros, shape])
    out["rq_none_codes_f32"] = codes0.numpy()
    sb, zb = scales.to(torch.bfloat16), zeros.to(torch.bfloat16)
    Wb = (W + torch.randn(64, 256, generator=g) * 0.003).to(torch.bfloat16)
    codes_b = ns["Qfunc_4bit_g_res"](Wb.clone(), Plain(), [sb, zb, shape])
    out["rq_none_w_bf16"] = f32(Wb)
    out["rq_none_codes_bf16"] = codes_b.numpy()

    # --- a3 dequant, fp32 and bf16 qparams ----------------------------------
    out["dq_f32"] = f32(ns["DeQfunc_4bit_g"](codes0, [scales, zeros, shape], torch.float32))
    out["dq_bf16"] = f32(ns["DeQfunc_4bit_g"](codes0, [sb, zb, shape], torch.bfloat16))

    # --- a12 uniform codec with real noise -----------------------------------
    r = torch.rand(2048, generator=g) - 0.5
    r[:8] = torch.tensor([-0.5, 0.5, 0.0, 0.46875, 0.499999, -0.499999, 0.25, -0.03125])
    torch.manual_seed(77)
    words, adj = ns["python_quant_linear"](r.clone())
    torch.manual_seed(77)
    noise = torch.empty(2048).uniform_(-0.5, 0.5)
    out["u16_r"], out["u16_noise"] = f32(r), f32(noise)
    out["u16_words"], out["u16_carry"] = words.numpy(), f32(adj)
    out["u16_decode"] = f32(ns["python_dequant_linear"](words)).reshape(-1)

    # --- a6 with the residual codec: config-1 style step, fp32 ---------------
    # latent = dequant(codes0) + delta ; requantize with a12 as the codec
    Wd = ns["DeQfunc_4bit_g"](codes0, [scales, zeros, shape], torch.float32)
    delta = torch.randn(64, 256, generator=g) * 1e-4
    lat = Wd + delta
    h = ResidualTensor(); h.noise_seed = 4321
    codes1 = ns["Qfunc_4bit_g_res"](lat.clone(), h, [scales, zeros, shape])
    torch.manual_seed(4321)
    noise1 = torch.empty(64 * 256).uniform_(-0.5, 0.5)
    out["c1_delta"], out["c1_noise1"] = f32(delta), f32(noise1)
    out["c1_codes0"], out["c1_codes1"] = codes0.numpy(), codes1.numpy()
    out["c1_words1"] = h.residual_int.numpy()
    # second step: latent = residual.add(dequant(codes1)) + delta2  (utils/quant.py:831-837)
    res_fp = ns["python_dequant_linear"](h.residual_int)
    lat2 = (res_fp.view(-1, 128) * scales).to(torch.float32).view(shape).add(
        ns["DeQfunc_4bit_g"](codes1, [scales, zeros, shape], torch.float32))
    delta2 = torch.randn(64, 256, generator=g) * 1e-4
    lat2 = lat2 + delta2
    h2 = ResidualTensor(); h2.noise_seed = 999
    codes2 = ns["Qfunc_4bit_g_res"](lat2.clone(), h2, [scales, zeros, shape])
    torch.manual_seed(999)
    noise2 = torch.empty(64 * 256).uniform_(-0.5, 0.5)
    out["c1_delta2"], out["c1_noise2"] = f32(delta2), f32(noise2)
    out["c1_codes2"], out["c1_words2"] = codes2.numpy(), h2.residual_int.numpy()
    X = torch.randn(32, 256, generator=g)
    out["c1_x"] = f32(X)
    out["c1_y"] = f32(X.mm(ns["DeQfunc_4bit_g"](codes2, [scales, zeros, shape], torch.float32).t()))

    # --- a13 A8W8 requantize with the residual codec, fp32 -------------------
    W8 = torch.randn(32, 128, generator=g) * 0.02
    qs = (W8.abs().amax(dim=1, keepdim=True) / 127.0)
    h8 = ResidualTensor(); h8.noise_seed = 555
    c8 = ns["Qfunc_8bit_res"](W8.clone(), h8, qs)
    torch.manual_seed(555)
    out["a8_noise"] = f32(torch.empty(32 * 128).uniform_(-0.5, 0.5))
    out["a8_w"], out["a8_qscales"] = f32(W8), f32(qs.reshape(-1))
    out["a8_codes"], out["a8_words"] = c8.numpy(), h8.residual_int.numpy()
    out["a8_codes_none"] = ns["Qfunc_8bit_res"](W8.clone(), None, qs).numpy()

    # --- C.6 optimizer-state codec ------------------------------------------
    st = torch.randn(4096, generator=g) * 1e-3
    q8, (sc, tm) = ns["Qfunc_8bit_opt"](st.clone(), blocksize=2)
    out["o8_x"], out["o8_q"] = f32(st), q8.numpy()
    out["o8_scale"], out["o8_tmax"] = f32(sc.reshape(-1)), f32(tm.reshape(-1))
    out["o8_deq"] = f32(ns["DeQfunc_8bit_opt"](q8, [sc, tm]))

    # --- a23 per-token activation quantizer (fake-quant output, fp32) -------
    A = torch.randn(16, 256, generator=g)
    A[:, 7] *= 20.0
    out["aq_x"] = f32(A)
    out["aq_fake"] = f32(ql["quantize_activation_per_token_absmax"](A.clone()))

    # --- MyAdam.update_step (utils/quant.py:1062-1148) on one A16W4 parameter, fp32 gradients, CPU states ----
    # lbit=16: the latent is a full-precision copy (no residual codec), so the Adam arithmetic, the 8-bit state
    # codec and the requantize are exercised exactly as the reference executes them.
    ad = slice_module(qpath, {"MyAdam", "QuantTensor", "GradientQTensor", "prodx", "python_compress", "python_decompress",
                              "Qfunc_8bit_opt", "DeQfunc_8bit_opt", "GROUPSIZE", "Qfunc_4bit_g_res", "DeQfunc_4bit_g",
                              "Qfunc_8bit_res"}, {"ResidualTensor": ResidualTensor, "warnings": __import__("warnings")})
    Na, Ka = 128, 512                                # 65536 elements: uint8 states, 32 blocks of 2048
    Wa = (torch.randn(Na, Ka, generator=g) * 0.02).to(torch.bfloat16).float()
    qa = qz["Quantizer"]()
    qa.configure(4, perchannel=True, sym=False, mse=False)
    qa.find_params(Wa.view(-1, 128), weight=True)
    sa = qa.scale.reshape(-1, 1).to(torch.bfloat16)
    za = qa.zero.reshape(-1, 1).to(torch.bfloat16)
    pt = ad["QuantTensor"]([Na, Ka], wbit=4, gbit=16, lbit=16)
    codes_a = ad["Qfunc_4bit_g_res"](Wa.to(torch.bfloat16), pt.residual, [sa, za, [Na, Ka]])
    pt.set_value(codes_a, [sa, za, [Na, Ka]])
    out["adam_w"], out["adam_scales"], out["adam_zeros"] = f32(Wa), f32(sa.reshape(-1)), f32(za.reshape(-1))
    out["adam_codes0"] = codes_a.numpy()
    opt = ad["MyAdam"]([{"params": [pt], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, cpu=True)
    for step in range(3):
        gr = torch.randn(Na, Ka, generator=g) * 1e-2
        pt.grad = gr.clone()
        group = opt.param_groups[0]
        if len(opt.state[pt]) == 0:
            opt.init_state(group, pt, 0, 0)
        opt.update_step(group, pt, 0, 0)
        st_ = opt.state[pt]
        out[f"adam_grad{step}"] = f32(gr)
        out[f"adam_codes{step + 1}"] = pt.data.numpy()
        out[f"adam_latent{step + 1}"] = f32(pt.residual.data)
        out[f"adam_state1_{step + 1}"] = st_["state1"].numpy()
        out[f"adam_state2_{step + 1}"] = st_["state2"].numpy()
        for k in ("qmap1", "absmax1", "qmap2", "absmax2"):
            out[f"adam_{k}_{step + 1}"] = f32(st_[k].reshape(-1))

    # --- PTQ packers (PTQ/quant/quant_linear.py:304-477, 578-692): checkpoint producers --------------------
    pq = slice_module(os.path.join(ref, "PTQ", "quant", "quant_linear.py"),
                      {"QuantLinearGPTQ", "QuantLinearA16W4", "QuantLinearA8W8", "python_compress", "python_decompress"})
    Np, Kp = 128, 256
    lin = torch.nn.Linear(Kp, Np, bias=True)
    lin.weight.data = (torch.randn(Np, Kp, generator=g) * 0.02)
    lin.bias.data = torch.randn(Np, generator=g) * 0.1
    qp_ = qz["Quantizer"]()
    qp_.configure(4, perchannel=True, sym=False, mse=False)
    qp_.find_params(lin.weight.data.view(-1, 128), weight=True)
    sc_g = qp_.scale.reshape(Np, Kp // 128).clone()          # [N, G] as PTQ/run.py:18-41 hands them over
    zr_g = qp_.zero.reshape(Np, Kp // 128).clone()
    out["ptq_w"], out["ptq_bias"] = f32(lin.weight.data), f32(lin.bias.data)
    out["ptq_scale"], out["ptq_zero"] = f32(sc_g), f32(zr_g)
    gq = pq["QuantLinearGPTQ"](4, 128, Kp, Np, True)
    gq.pack(lin, sc_g.clone(), zr_g.clone(), None)
    out["gptq_qweight"], out["gptq_qzeros"] = gq.qweight.numpy(), gq.qzeros.numpy()
    out["gptq_scales"], out["gptq_g_idx"] = f32(gq.scales), gq.g_idx.numpy()
    out["gptq_unpack"] = f32(gq.unpack(gq.qweight, gq.scales, gq.qzeros))
    a4 = pq["QuantLinearA16W4"](4, 128, Kp, Np, True)
    a4.pack(lin, sc_g.clone(), zr_g.clone(), None)
    out["a16w4_qweight"] = a4.qweight.numpy()
    out["a16w4_scales"], out["a16w4_zeros"] = f32(a4.scales.reshape(-1)), f32(a4.zeros.reshape(-1))
    out["a16w4_unpack"] = f32(a4.unpack(a4.qweight))
    qs_ = qz["Quantizer"]()
    qs_.configure(8, perchannel=True, sym=True, mse=False)
    qs_.find_params(lin.weight.data, weight=True)
    a8 = pq["QuantLinearA8W8"](8, -1, Kp, Np, True)
    a8.pack(lin, qs_.scale.clone(), qs_.zero.clone(), None)
    out["a8w8_qweight"], out["a8w8_qzeros"] = a8.qweight.numpy(), a8.qzeros.numpy().astype(np.int32)
    out["a8w8_scales"] = f32(a8.scales.reshape(-1))

    # --- a14: the activation quantizer inside QLinearFunctionA8W8_dynamic.forward (utils/quant.py:258-272) -----
    # The class body is executed as written; the external int8 GEMM is replaced by a recorder that keeps its
    # arguments (the quantized activations, the bias/qscales operand and alpha = clampv/127).
    seen = {}

    def linear_a8_w8_bbf16_obf16(x8, w8, bias_over_scale, alpha):
        seen["x8"], seen["alpha"], seen["bias_arg"] = x8.clone(), alpha.clone(), bias_over_scale.clone()
        return torch.zeros(x8.shape[0], w8.shape[0], dtype=bias_over_scale.dtype)

    dyn = slice_module(qpath, {"QLinearFunctionA8W8_dynamic"},
                       {"linear_a8_w8_bbf16_obf16": linear_a8_w8_bbf16_obf16, "dict_temp": []})

    class Ctx:
        def save_for_backward(self, *a):
            pass
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        Xa = torch.randn(24, 256, generator=g)
        Xa[:, 11] *= 20.0
        Xa = Xa.to(dt)
        w8 = torch.randint(-128, 128, (16, 256), generator=g, dtype=torch.int8)
        qsc = (torch.rand(16, generator=g) * 1e-2 + 1e-3).to(dt)
        bia = (torch.randn(16, generator=g) * 0.1).to(dt)
        dyn["QLinearFunctionA8W8_dynamic"].forward(Ctx(), Xa, w8, (None, qsc), bia)
        out[f"pt_x_{tag}"] = f32(Xa)
        out[f"pt_x8_{tag}"] = seen["x8"].numpy()
        out[f"pt_clampv_{tag}"] = f32(Xa.max().reshape(1))
        out[f"pt_alpha_{tag}"] = f32(seen["alpha"].reshape(1))

    # --- GradientQTensor (utils/quant.py:846-921): set_value then two add_ calls, fp32 and bf16, seeded noise ----------
    gq = slice_module(qpath, {"GradientQTensor"})
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        acc = gq["GradientQTensor"]([24, 256], bit=8)
        for it in range(3):
            fd = (torch.randn(24, 256, generator=g) * (1e-3 if it else 2e-3)).to(dt)
            if it == 0:
                fd[3] = 0.0                                   # an all-zero row: the 1e-5 floor of the scale
            seed = 900 + it
            torch.manual_seed(seed)
            if it == 0:
                acc.set_value(fd.clone())
            else:
                acc.add_(fd.clone())
            torch.manual_seed(seed)
            out[f"gq_noise{it}_{tag}"] = f32(torch.empty(24, 256, dtype=dt).uniform_(-0.5, 0.5))
            out[f"gq_f{it}_{tag}"] = f32(fd)
            out[f"gq_q{it}_{tag}"] = acc.qdata.numpy().copy()
        out[f"gq_scale_{tag}"] = f32(acc.scale.reshape(-1))
        out[f"gq_value_{tag}"] = f32(acc.get_value())

    # --- a9-a11: the CUDA residual codecs, from the reference's own kernel text compiled for the CPU ------------
    # (oracle/build_ref.py: no GPU launch).  Built with and without FMA contraction; the fixtures are the FMA
    # build (nvcc's default), `rc_variants_agree` records whether the other build produced the same bytes.
    import ctypes as C
    sys.path.insert(0, os.path.dirname(os.path.dirname(OUT)))
    import oracle as orc
    from oracle import build_ref
    build_ref.build(ref)
    libs = {v: C.CDLL(build_ref.lib_path(v)) for v in ("fma", "nofma")}

    def p_(a):
        return a.ctypes.data_as(C.c_void_p)

    def bf(a16):
        return (a16.astype(np.uint32) << 16).view(np.float32)
    pats, _ = orc.bf16_codec_domain()
    all_nibbles = np.array([0x01234567, 0x89abcdef - (1 << 32)], dtype=np.int64).astype(np.int32)
    agree = True
    for mu in range(4):
        k1, b1, k2, b2, k3 = orc.curve_args(mu)
        args = (k1, C.c_float(b1), k2, C.c_float(b2), k3)
        xg = orc.f32_codec_grid(mu)
        res = {}
        for v, L in libs.items():
            r = {}
            x = pats.copy(); y = np.empty(x.size // 8, np.int32); c8 = np.empty(8, np.float32)
            L.ref_quant_bf16(p_(x), p_(y), *args, y.size, p_(c8))
            r["q_bf16_words"], r["q_bf16_flags"], r["q_consts"] = y, np.packbits(bf(x) != 0), c8
            x = xg.copy(); y = np.empty(x.size // 8, np.int32)
            L.ref_quant_f32(p_(x), p_(y), *args, y.size, None)
            r["q_f32_words"], r["q_f32_flags"] = y, np.packbits(x != 0)
            assert set(np.unique(x)) <= {0.0, 1.0}
            o16 = np.empty(16, np.uint16); c7 = np.empty(7, np.float32)
            L.ref_dequant_bf16(p_(all_nibbles), p_(o16), *args, 2, p_(c7))
            o32 = np.empty(16, np.float32)
            L.ref_dequant_f32(p_(all_nibbles), p_(o32), *args, 2, None)
            r["dq_bf16"], r["dq_f32"], r["dq_consts"] = bf(o16), o32, c7
            res[v] = r
        for k, a in res["fma"].items():
            out[f"rc_{k}_mu{mu}"] = a
            agree &= np.array_equal(a, res["nofma"][k])
    xg = orc.f32_codec_grid(0, seed=77)
    res = {}
    for v, L in libs.items():
        r = {}
        x = pats.copy(); y = np.empty(x.size // 8, np.int32)
        L.ref_uniform_quant_bf16(p_(x), p_(y), y.size)
        r["uq_bf16_words"], r["uq_bf16_flags"] = y, np.packbits(bf(x) != 0)
        x = xg.copy(); y = np.empty(x.size // 8, np.int32)
        L.ref_uniform_quant_f32(p_(x), p_(y), y.size)
        r["uq_f32_words"], r["uq_f32_flags"] = y, np.packbits(x != 0)
        x = xg.copy(); y = np.empty(x.size // 8, np.int32)
        L.ref_uniform_quant_s_f32(p_(x), p_(y), y.size)
        r["uqs_f32_words"], r["uqs_f32_flags"] = y, np.packbits(x != 0)
        o16 = np.empty(16, np.uint16); o32 = np.empty(16, np.float32)
        L.ref_uniform_dequant_bf16(p_(all_nibbles), p_(o16), 2)
        L.ref_uniform_dequant_f32(p_(all_nibbles), p_(o32), 2)
        r["udq_bf16"], r["udq_f32"] = bf(o16), o32
        res[v] = r
    for k, a in res["fma"].items():
        out[f"rc_{k}"] = a
        agree &= np.array_equal(a, res["nofma"][k])
    out["rc_variants_agree"] = np.array([agree])
    out["rc_all_nibbles"] = all_nibbles

    np.savez_compressed(os.path.join(OUT, "reference_vectors.npz"), **out)
    print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(OUT, "reference_vectors.npz")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/gen_golden.py /path/to/latentQ_LLM")
    main(sys.argv[1])
