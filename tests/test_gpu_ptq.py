"""Checkpoint-side modules (mirror of PTQ/quant/quant_linear.py) against vectors produced by the reference's own
`pack` / `unpack` methods, and the GPTQ-layout GEMM entry points."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _linear(golden):
    lin = torch.nn.Linear(256, 128, bias=True)
    lin.weight.data = torch.from_numpy(golden["ptq_w"])
    lin.bias.data = torch.from_numpy(golden["ptq_bias"])
    return lin


def test_gptq_pack_unpack_and_gemm(golden):
    from latentq_llm_b200 import ops, ptq
    m = ptq.QuantLinearGPTQ(4, 128, 256, 128, True).cuda()
    m.pack(_linear(golden), torch.from_numpy(golden["ptq_scale"]), torch.from_numpy(golden["ptq_zero"]), None)
    assert m.qweight.dtype == torch.int32 and np.array_equal(m.qweight.cpu().numpy(), golden["gptq_qweight"])
    assert np.array_equal(m.qzeros.cpu().numpy(), golden["gptq_qzeros"])
    assert np.array_equal(m.scales.float().cpu().numpy(), golden["gptq_scales"])
    assert np.array_equal(m.g_idx.cpu().numpy(), golden["gptq_g_idx"])
    W = m.unpack(m.qweight, m.scales, m.qzeros)
    assert np.array_equal(W.cpu().numpy(), golden["gptq_unpack"])
    # layout conversion round trip
    codes = ops.gptq_to_nibblepair(m.qweight, 128, 256)
    assert torch.equal(ops.nibblepair_to_gptq(codes, 128, 256), m.qweight)
    # GEMM entry points of the GPTQ layout (fp16 in / out like the reference)
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(40, 256, device="cuda", generator=g).half().requires_grad_(True)
    y = m(x)
    ref = x.detach().float() @ W.t() + m.bias.float()
    assert y.dtype == torch.float16 and float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2
    dy = torch.randn(40, 128, device="cuda", generator=g).half()
    y.backward(dy)
    ref = dy.float() @ W
    assert float((x.grad.float() - ref).abs().max() / ref.abs().max()) < 1e-2
    # the layout conversion is cached per set of buffers: the second call converts nothing
    n_cached = len(ptq._GPTQ_CACHE)
    m(x.detach())
    assert len(ptq._GPTQ_CACHE) == n_cached
    bad = m.g_idx.clone(); bad[:5] = 1                       # 123 / 133 members: not a grouping the layout can hold
    with pytest.raises(NotImplementedError):
        ptq.matmul248(x.detach(), m.qweight, m.scales, m.qzeros, bad, 4, 15)


def test_gptq_gemm_with_act_order_g_idx(golden):
    """A general g_idx (input feature k takes the scale / zero row g_idx[k], PTQ/quant/quant_linear.py:113-122), as
    act-order GPTQ checkpoints carry it: forward and grad-input against the module's own `unpack`."""
    from latentq_llm_b200 import ptq
    K, N, gs = 512, 256, 128
    g = torch.Generator().manual_seed(5)
    lin = torch.nn.Linear(K, N, bias=False)
    lin.weight.data = torch.randn(N, K, generator=g) * 0.02
    order = torch.randperm(K, generator=g)
    g_idx = torch.empty(K, dtype=torch.int32)
    g_idx[order] = (torch.arange(K) // gs).to(torch.int32)   # feature order[i] belongs to group i // gs
    # per-group min/max parameters over the features of each group
    W = lin.weight.data
    scale, zero = torch.empty(N, K // gs), torch.empty(N, K // gs)
    for gi in range(K // gs):
        blk = W[:, g_idx == gi]
        lo, hi = blk.amin(1).clamp(max=0), blk.amax(1).clamp(min=0)
        scale[:, gi] = (hi - lo) / 15
        zero[:, gi] = torch.round(-lo / scale[:, gi])
    # the layer as a quantizer hands it to `pack`: weights already on the grid (codes clamped to [0, 15])
    gi = g_idx.long()
    sc_k, zr_k = scale.half().float()[:, gi], zero[:, gi]                        # [N, K]
    lin.weight.data = sc_k * (torch.clamp(torch.round(W / sc_k) + zr_k, 0, 15) - zr_k)
    m = ptq.QuantLinearGPTQ(4, gs, K, N, False).cuda()
    m.pack(lin, scale, zero, g_idx.cuda())
    Wd = m.unpack(m.qweight, m.scales, m.qzeros)             # honours g_idx
    assert float((Wd.cpu() - lin.weight.data).abs().max()) < 2e-2 * float(scale.max())     # fp16 scale and product rounding
    for M in (4, 48):                                        # decode route and tensor-core route
        x = torch.randn(M, K, device="cuda").half().requires_grad_(True)
        y = m(x)
        ref = x.detach().float() @ Wd.t()
        assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2
        dy = torch.randn(M, N, device="cuda").half()
        y.backward(dy)
        ref = dy.float() @ Wd
        assert float((x.grad.float() - ref).abs().max() / ref.abs().max()) < 1e-2


def test_a16w4_and_a8w8_packers(golden):
    from latentq_llm_b200 import ptq
    a4 = ptq.QuantLinearA16W4(4, 128, 256, 128, True)
    a4.pack(_linear(golden), torch.from_numpy(golden["ptq_scale"]), torch.from_numpy(golden["ptq_zero"]), None)
    assert a4.qweight.dtype == torch.int8 and np.array_equal(a4.qweight.cpu().numpy(), golden["a16w4_qweight"])
    assert np.array_equal(a4.scales.float().cpu().numpy().ravel(), golden["a16w4_scales"])
    assert np.array_equal(a4.zeros.float().cpu().numpy().ravel(), golden["a16w4_zeros"])
    W = a4.unpack(a4.qweight)
    assert np.array_equal(W.float().cpu().numpy(), golden["a16w4_unpack"])
    x = torch.randn(24, 256, device="cuda").half()
    ref = x.float() @ W.float().t() + a4.bias.float()
    assert float((a4(x).float() - ref).abs().max() / ref.abs().max()) < 1e-2
    # A8W8: symmetric per-channel uint8 weights with zero point 128
    import oracle as orc
    w = golden["ptq_w"]
    s, z = orc.find_qparams(w, 256, 255, True)
    a8 = ptq.QuantLinearA8W8(8, -1, 256, 128, True)
    a8.pack(_linear(golden), torch.from_numpy(s), torch.from_numpy(z), None)
    assert a8.qweight.dtype == torch.uint8 and np.array_equal(a8.qweight.cpu().numpy(), golden["a8w8_qweight"])
    assert np.array_equal(a8.qzeros.cpu().numpy().astype(np.int32), golden["a8w8_qzeros"])
    assert np.array_equal(a8.scales.float().cpu().numpy().ravel(), golden["a8w8_scales"])
    a8.clampv = 4.0
    y = a8(x.to(torch.bfloat16))
    ref = x.float().clamp(-4, 4) @ a8.unpack(a8.qweight).float().t() + a8.bias.float()
    assert float((y.float() - ref).norm() / ref.norm()) < 3e-2


def test_per_token_fake_quant(golden):
    from latentq_llm_b200 import ptq
    t = torch.from_numpy(golden["aq_x"]).cuda().to(torch.bfloat16)
    out = ptq.quantize_activation_per_token_absmax(t.clone())
    import oracle as orc
    q, s = orc.act_quant_per_token(t.float().cpu().numpy(), math_bf16=True)
    want = orc.bf16_round(q.astype(np.float32) * s[:, None])
    assert np.array_equal(out.float().cpu().numpy(), want)


def test_make_quant_linear_surgery_and_warmup():
    """Model surgery of the PTQ side: named linears are replaced by packed layers of the configured layout, calibration
    statistics travel, untouched layers stay, and a packed GPTQ model runs after the one-time warm-up."""
    import torch.nn as nn
    from latentq_llm_b200 import ptq

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2, self.keep = nn.Linear(256, 512), nn.Linear(512, 256, bias=False), nn.Linear(256, 64)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([Block(), Block()])

    names = {"blocks.0.fc1": None, "blocks.0.fc2": None, "blocks.1.fc1": None}
    for method, cls in (("gptq", ptq.QuantLinearGPTQ), ("a16w4", ptq.QuantLinearA16W4)):
        net = Net()
        ptq.config["method"] = method
        ptq.make_quant_linear(net, names, 4, 128)
        assert isinstance(net.blocks[0].fc1, cls) and isinstance(net.blocks[0].fc2, cls) and isinstance(net.blocks[1].fc1, cls)
        assert isinstance(net.blocks[1].fc2, nn.Linear) and isinstance(net.blocks[0].keep, nn.Linear)
        assert net.blocks[0].fc1.name == "blocks.0.fc1" and net.blocks[0].fc2.bias is None
    ptq.config["method"] = "gptq"
    net = Net()
    net.blocks[0].fc1.inp_absmax = torch.full((256,), 2.0, dtype=torch.float16)
    ptq.make_quant_linear(net, {"blocks.0.fc1": None}, 8, -1)
    assert isinstance(net.blocks[0].fc1, ptq.QuantLinearA8W8) and float(net.blocks[0].fc1.inp_absmax.max()) == 2.0
    assert ptq.QuantLinear0 is ptq.QuantLinearGPTQ and ptq.QuantLinear1 is ptq.QuantLinearA8W8 and ptq.QuantLinear2 is ptq.QuantLinearA16W4
    # a packed GPTQ layer inside a model: warm-up visits each distinct (K, N) once
    net = Net().cuda()
    ptq.make_quant_linear(net, {"blocks.0.fc1": None, "blocks.1.fc1": None}, 4, 128)
    net = net.cuda()
    assert ptq.autotune_warmup_linear(net, transpose=True) == 1
