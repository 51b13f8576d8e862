"""Fused optimizer step (`lq_adam_a16w4_step`, `lq_adam_dense_multi`) against the op-by-op MyAdam.update_step route,
which `test_gpu_module.py::test_myadam_matches_reference_steps` pins to the reference's own optimizer output.
Bit-exact: packed codes, residual words, 8-bit states and their block parameters, dense bf16 parameters and states."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _quant_param(Q, N, K, seed):
    from latentq_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    s, z = ops.find_qparams(w, 128, 15, False)
    layer = Q.QLinearA16W4(K, N, bias=False, lbit=4, gbit=16)
    layer.zeros.data = z.view(-1, 1).to(torch.bfloat16)
    layer.scales.data = s.view(-1, 1).to(torch.bfloat16)
    codes, _ = ops.a16w4_requant(w, layer.scales.data.view(-1).contiguous(), layer.zeros.data.view(-1).contiguous(),
                                 ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16))
    layer.weight.set_value(codes, [layer.scales, layer.zeros, layer.wshape])
    layer.to("cuda")
    return layer


def _same_state(sa, sb):
    for k in ("state1", "state2"):
        assert torch.equal(sa[k], sb[k]), k
    for k in ("qmap1", "absmax1", "qmap2", "absmax2"):
        assert torch.equal(sa[k].reshape(-1), sb[k].reshape(-1)), k
    assert sa["step"] == sb["step"]


@pytest.mark.parametrize("N,K", [(512, 1024), (520, 128), (2048, 2048)])   # 2048-element blocks, 128-element blocks, larger
def test_fused_quantized_step_is_bit_identical(N, K):
    from latentq_llm_b200 import quant as Q
    la, lb = _quant_param(Q, N, K, seed=5), _quant_param(Q, N, K, seed=5)
    pa, pb = la.weight, lb.weight
    assert torch.equal(pa.data, pb.data)
    oa = Q.MyAdam([{"params": [pa], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, fused=False)
    ob = Q.MyAdam([{"params": [pb], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, fused=True)
    g = torch.Generator(device="cuda").manual_seed(11)
    for t in range(5):
        scale = 10.0 ** (-(t % 3) - 1)                         # gradients of different magnitudes
        grad = (torch.randn(N, K, device="cuda", generator=g) * scale).to(torch.bfloat16)
        pa.grad, pb.grad = grad.clone(), grad.clone()
        oa.step(); ob.step()
        assert torch.equal(pa.data.view(torch.uint8), pb.data.view(torch.uint8)), f"codes differ at step {t}"
        assert torch.equal(pa.residual.residual_int, pb.residual.residual_int), f"residual words differ at step {t}"
        _same_state(oa.state[pa], ob.state[pb])
        assert pa.grad is None and pb.grad is None
        assert pb.residual.lock_mu == pa.residual.lock_mu and not pb.residual.init
    # the fused route ran (uint8 states were updated in place, no new tensors)
    assert ob.state[pb]["state1"].dtype == torch.uint8 and int(ob.state[pb]["state1"].max()) > 0


@pytest.mark.parametrize("gscale", [1e-2, 3e-4, 1e-5])       # different |m| / denom levels -> different curve levels
def test_fused_step_through_a_curve_refresh_step(gscale):
    """Steps on which the residual-curve level is refreshed (utils/quant.py:1107-1111) stay on the fused route: a
    read-only statistics kernel runs first, the level it selects is the one the step encodes with — as in the op-by-op
    route, whose codes, residual words, states and levels must come out identical."""
    from latentq_llm_b200 import quant as Q
    N, K = 512, 512
    la, lb = _quant_param(Q, N, K, seed=2), _quant_param(Q, N, K, seed=2)
    pa, pb = la.weight, lb.weight
    oa = Q.MyAdam([{"params": [pa], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, mu_updata_f=4, fused=False)
    ob = Q.MyAdam([{"params": [pb], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, mu_updata_f=4, fused=True)
    g = torch.Generator(device="cuda").manual_seed(4)
    start = pb.data.clone()
    for t in range(3):
        grad = (torch.randn(N, K, device="cuda", generator=g) * 1e-2).to(torch.bfloat16)
        pa.grad, pb.grad = grad.clone(), grad.clone()
        oa.step(); ob.step()
    assert not torch.equal(start, pb.data)
    # jump both optimizers past the step where the residual curve level is refreshed (step > 250, step % f == f-1)
    oa.state[pa]["step"] = ob.state[pb]["step"] = 253
    for t in range(7):                                          # steps 254 .. 260; refreshes at 255 and 259
        grad = (torch.randn(N, K, device="cuda", generator=g) * gscale).to(torch.bfloat16)
        pa.grad, pb.grad = grad.clone(), grad.clone()
        oa.step(); ob.step()
        assert pa.residual.mu == pb.residual.mu and pa.residual.lock_mu == pb.residual.lock_mu, t
        assert torch.equal(pa.data.view(torch.uint8), pb.data.view(torch.uint8)), t
        assert torch.equal(pa.residual.residual_int, pb.residual.residual_int), t
    _same_state(oa.state[pa], ob.state[pb])
    assert ob.op_by_op_steps == 0 and oa.op_by_op_steps == 10


def _a8w8_param(Q, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    layer = Q.QLinearA8W8(K, N, bias=False, lbit=4, gbit=16)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    qs = (w.abs().amax(dim=1, keepdim=True) / 127).to(torch.bfloat16)
    layer.qscales.data = qs
    w8 = torch.clamp(torch.round(w / qs.float()), -128, 127).to(torch.int8)
    layer.weight.set_value(w8, layer.qscales)
    layer.to("cuda")
    return layer


@pytest.mark.parametrize("N,K", [(192, 512), (520, 128), (256, 2048)])   # 2048-element, 128-element state blocks, long rows
def test_fused_a8w8_step_is_bit_identical(N, K):
    """`lq_adam_a8w8_step` (int8 latent weights, one scale per row) against the op-by-op route, including two steps
    that refresh the curve level (statistics per weight row)."""
    from latentq_llm_b200 import quant as Q
    la, lb = _a8w8_param(Q, N, K, seed=7), _a8w8_param(Q, N, K, seed=7)
    pa, pb = la.weight, lb.weight
    oa = Q.MyAdam([{"params": [pa], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, mu_updata_f=4, fused=False)
    ob = Q.MyAdam([{"params": [pb], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, mu_updata_f=4, fused=True)
    g = torch.Generator(device="cuda").manual_seed(13)
    for t in range(9):
        if t == 4:
            oa.state[pa]["step"] = ob.state[pb]["step"] = 253
        grad = (torch.randn(N, K, device="cuda", generator=g) * 10.0 ** (-(t % 3) - 2)).to(torch.bfloat16)
        pa.grad, pb.grad = grad.clone(), grad.clone()
        oa.step(); ob.step()
        assert torch.equal(pa.data, pb.data), f"codes differ at step {t}"
        assert torch.equal(pa.residual.residual_int, pb.residual.residual_int), f"residual words differ at step {t}"
        assert pa.residual.mu == pb.residual.mu and pa.residual.lock_mu == pb.residual.lock_mu
        _same_state(oa.state[pa], ob.state[pb])
    assert ob.op_by_op_steps == 0


def test_gradient_accumulator_kernel_vs_reference_vectors(golden):
    """GradientQTensor (utils/quant.py:846-921): set_value and two add_ calls with the noise the reference drew,
    against what the reference's class produced (fp32 and bf16), then the Philox-noise route against the oracle."""
    import numpy as np
    import oracle as orc
    from latentq_llm_b200 import ops
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        q = torch.empty((24, 256), dtype=torch.int8, device="cuda")
        sc = torch.empty(24, dtype=dt, device="cuda")
        for it in range(3):
            f = torch.from_numpy(golden[f"gq_f{it}_{tag}"]).cuda().to(dt)
            noise = torch.from_numpy(golden[f"gq_noise{it}_{tag}"]).cuda()
            ops.gradq_accumulate(f, q, sc, it == 0, ops.make_opts(dither=ops.DITHER_EXPLICIT, dither_buf=noise))
            assert np.array_equal(q.cpu().numpy(), golden[f"gq_q{it}_{tag}"]), (tag, it)
        assert np.array_equal(sc.float().cpu().numpy(), golden[f"gq_scale_{tag}"])
        assert np.array_equal(ops.gradq_dequant(q, sc).float().cpu().numpy(), golden[f"gq_value_{tag}"])
    # Philox noise: the library's stream, one block per 8 elements
    rng = np.random.default_rng(3)
    f = orc.bf16_round((rng.standard_normal((40, 1024)) * 1e-3).astype(np.float32))
    q = torch.empty((40, 1024), dtype=torch.int8, device="cuda")
    sc = torch.empty(40, dtype=torch.bfloat16, device="cuda")
    ops.gradq_accumulate(torch.from_numpy(f).cuda().to(torch.bfloat16), q, sc, True,
                         ops.make_opts(dither=ops.DITHER_PHILOX, seed=99, step=1, param_id=5))
    want_q, want_s = orc.gradq_accumulate(f, orc.philox_dither(99, (1 << 32) | 5, 40 * 1024 // 8).reshape(40, 1024), math_bf16=True)
    assert np.array_equal(q.cpu().numpy(), want_q) and np.array_equal(sc.float().cpu().numpy(), want_s)


def test_gradient_accumulator_class_in_the_hook_route():
    """QLinearA16W4 with gbit=8: the backward hook folds every micro-batch into the 8-bit accumulator, the optimizer
    reads it back (utils/quant.py:398-411, 1064-1065) and stays on the fused route."""
    from latentq_llm_b200 import quant as Q
    N, K, M = 256, 512, 32
    layer = _quant_param(Q, N, K, seed=3)
    layer.weight.grad = Q.GradientQTensor([N, K], bit=8, seed=1)
    layer.add_hook()
    opt = Q.MyAdam([{"params": [layer.weight], "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8)
    g = torch.Generator(device="cuda").manual_seed(8)
    before = layer.weight.data.clone()
    dense = torch.zeros(N, K, device="cuda")
    for mb in range(3):
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
        y = layer(x)
        y.backward(torch.ones_like(y) * 1e-2)
        dense += (torch.ones(M, N, device="cuda") * 1e-2).t() @ x.detach().float()
    acc = layer.weight.grad
    assert isinstance(acc, Q.GradientQTensor) and acc.acc_ite == 3 and acc.qdata.dtype == torch.int8
    got = acc.get_value().float()
    assert float((got - dense).abs().max()) <= 3.0 * float(acc.scale.float().max())     # within a few quantization steps
    opt.step()
    # (a first step moves every weight by lr = 1e-3, a fraction of a code step: it lands in the residual words)
    res = layer.weight.residual
    assert opt.op_by_op_steps == 0 and acc.acc_ite == 0 and not res.init
    assert int((res.residual_int.view(-1) != 0x88888888 - (1 << 32)).sum()) > res.residual_int.numel() // 2
    assert torch.equal(before, layer.weight.data)


def test_fused_dense_multi_is_bit_identical():
    from latentq_llm_b200 import quant as Q
    shapes = [(2048,), (8192,), (7,), (33, 5), (1,), (255, 255)]
    g = torch.Generator(device="cuda").manual_seed(9)
    A = [torch.nn.Parameter((torch.randn(*s, device="cuda", generator=g) * 0.5).to(torch.bfloat16)) for s in shapes]
    B = [torch.nn.Parameter(a.detach().clone()) for a in A]
    oa = Q.MyAdam([{"params": A, "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, fused=False)
    ob = Q.MyAdam([{"params": B, "weight_decay": 0.0}], lr=1e-3, betas=(0.9, 0.95), obit=8, fused=True)
    for t in range(6):
        for a, b in zip(A, B):
            gr = (torch.randn(*a.shape, device="cuda", generator=g) * 10.0 ** (-(t % 4))).to(torch.bfloat16)
            a.grad, b.grad = gr.clone(), gr.clone()
        oa.step(); ob.step()
        for i, (a, b) in enumerate(zip(A, B)):
            assert torch.equal(a.data, b.data), (t, i)
            assert torch.equal(oa.state[a]["state1"], ob.state[b]["state1"]), (t, i)
            assert torch.equal(oa.state[a]["state2"], ob.state[b]["state2"]), (t, i)
            assert b.grad is None
    assert ob._dense_tables[0].n == len(shapes)


def test_fused_entry_point_rejects_bad_arguments():
    from latentq_llm_b200 import _lib as L, ops
    n = 4096
    codes = torch.zeros(n // 2, dtype=torch.int8, device="cuda"); words = torch.zeros(n // 8, dtype=torch.int32, device="cuda")
    grad = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    s = torch.ones(n // 128, dtype=torch.bfloat16, device="cuda"); z = torch.zeros_like(s)
    st = torch.zeros(n, dtype=torch.uint8, device="cuda")
    blk = torch.zeros(n // 2048, dtype=torch.float32, device="cuda")
    h = ops.make_adam_hyper(0.9, 0.95, 1e-8, 1e-3)
    o = ops.make_opts(codec=ops.CODEC_NONE)                     # the fused step needs a residual codec
    with pytest.raises(L.LatentQError) as e:
        ops.adam_a16w4_step(codes, words, grad, s, z, st, blk, blk.clone(), st.clone(), blk.clone(), blk.clone(), h, o)
    assert e.value.status == L.LQ_EUNSUPPORTED
    o = ops.make_opts(math_dtype=torch.float32)                 # chain dtype must be the gradient's
    with pytest.raises(L.LatentQError) as e:
        ops.adam_a16w4_step(codes, words, grad, s, z, st, blk, blk.clone(), st.clone(), blk.clone(), blk.clone(), h, o)
    assert e.value.status == L.LQ_EUNSUPPORTED


@pytest.mark.parametrize("generic", [False, True])                # table-driven fast kernel / generic kernel
@pytest.mark.parametrize("n_rows,K", [(32, 2048), (40, 128)])     # 2048-element and 128-element state blocks
def test_fused_quantized_step_matches_oracle(n_rows, K, generic, monkeypatch):
    """The CUDA kernel against the CPU restatement of the GPU evaluation order, two consecutive steps (the second
    one decodes a live residual and non-trivial 8-bit states)."""
    import numpy as np
    import oracle as orc
    from latentq_llm_b200 import ops
    if generic:
        monkeypatch.setenv("LQ_REQUANT_GENERIC", "1")
    else:
        monkeypatch.delenv("LQ_REQUANT_GENERIC", raising=False)
    n = n_rows * K
    block = 2048 if n % 2048 == 0 else 128
    g = torch.Generator(device="cuda").manual_seed(21)
    w = (torch.randn(n, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    s, z = ops.find_qparams(w, 128, 15, False)
    s, z = s.to(torch.bfloat16).contiguous(), z.to(torch.bfloat16).contiguous()
    codes, _ = ops.a16w4_requant(w, s, z, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16))
    words = torch.zeros(n // 8, dtype=torch.int32, device="cuda")
    st1 = torch.zeros(n, dtype=torch.uint8, device="cuda"); st2 = torch.zeros_like(st1)
    sc1 = torch.full((n // block,), 1e-10, dtype=torch.float32, device="cuda"); sc2 = sc1.clone()
    tm1 = torch.zeros(n // block, dtype=torch.float32, device="cuda"); tm2 = tm1.clone()
    host = dict(codes=codes.cpu().numpy(), words=words.cpu().numpy(), st1=st1.cpu().numpy(), sc1=sc1.cpu().numpy(),
                tm1=tm1.cpu().numpy(), st2=st2.cpu().numpy(), sc2=sc2.cpu().numpy(), tm2=tm2.cpu().numpy())
    sf, zf = s.float().cpu().numpy(), z.float().cpu().numpy()
    for t in (1, 2):
        grad = (torch.randn(n, device="cuda", generator=g) * 1e-2).to(torch.bfloat16)
        step_size = 1e-3 * (1 - 0.95 ** t) ** 0.5 / (1 - 0.9 ** t)
        ops.adam_a16w4_step(codes, words, grad, s, z, st1, sc1, tm1, st2, sc2, tm2,
                            ops.make_adam_hyper(0.9, 0.95, 1e-8, step_size),
                            ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, math_dtype=torch.bfloat16,
                                          res_round_bf16=True, has_residual=(t > 1)))
        out = orc.adam_a16w4_step(host["codes"], host["words"], grad.float().cpu().numpy(), sf, zf,
                                  host["st1"], host["sc1"], host["tm1"], host["st2"], host["sc2"], host["tm2"],
                                  beta1=0.9, beta2=0.95, eps=1e-8, step_size=step_size, math_bf16=True,
                                  has_residual=(t > 1))
        host = dict(zip(("codes", "words", "st1", "sc1", "tm1", "st2", "sc2", "tm2"), out))
        for name, dev in (("codes", codes), ("words", words), ("st1", st1), ("sc1", sc1), ("tm1", tm1),
                          ("st2", st2), ("sc2", sc2), ("tm2", tm2)):
            assert np.array_equal(dev.cpu().numpy().ravel(), np.asarray(host[name]).ravel()), (t, name)
