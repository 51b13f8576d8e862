"""GPU parity of the tcgen05 GEMMs.

int8: accumulators are compared bit for bit with the oracle (small shapes) and with an exact
integer matmul on the device (benchmark shapes).  A16W4: outputs within 1e-2 relative of the
reference's dequantize-then-matmul (tolerance stated by the target), measured as
max|err| / max|ref| and as a relative Frobenius error."""
import numpy as np
import pytest
import torch

import oracle as orc

pytestmark = pytest.mark.gpu
RTOL = 1e-2


@pytest.fixture(scope="module")
def ops():
    from latentq_llm_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def _no_device_timeout():
    yield
    from latentq_llm_b200 import _lib
    assert _lib.lib.lq_gemm_device_status(1) == 0, "a bounded device-side wait expired"


@pytest.fixture(params=["tmem", "smem"])
def a_operand(request, monkeypatch):
    """Where the dequantised weight tile lives for the MMA: tensor memory (default) or shared memory."""
    monkeypatch.setenv("LQ_GEMM_A_OPERAND", request.param)
    return request.param


def make_w4_layer(ops, N, K, seed, group=128):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    s, z = ops.find_qparams(w, group, 15, False)
    sb, zb = s.to(torch.bfloat16), z.to(torch.bfloat16)
    codes, _ = ops.a16w4_requant(w, sb, zb, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16), group=group)
    return codes, sb, zb


def rel_err(got, ref):
    got, ref = got.double(), ref.double()
    return float((got - ref).abs().max() / ref.abs().max()), float((got - ref).norm() / ref.norm())


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 256, 512), (33, 192, 384), (128, 128, 256), (200, 320, 1024)])
def test_a16w4_fwd_small_vs_oracle(ops, a_operand, M, N, K):
    codes, sb, zb = make_w4_layer(ops, N, K, seed=M + N)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    y = ops.gemm_a16w4_fwd(x, codes, sb, zb, bias, N, K)
    ref = orc.gemm_a16w4(x.float().cpu().numpy(), codes.cpu().numpy(), sb.float().cpu().numpy(), zb.float().cpu().numpy(),
                         N, K, bias=bias.float().cpu().numpy())
    e_max, e_fro = rel_err(y.cpu(), torch.from_numpy(ref))
    assert e_max < RTOL and e_fro < RTOL, (e_max, e_fro)


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 256, 512), (33, 192, 384), (128, 128, 256), (200, 320, 1024)])
def test_a16w4_dgrad_small_vs_oracle(ops, a_operand, M, N, K):
    codes, sb, zb = make_w4_layer(ops, N, K, seed=M + K)
    g = torch.Generator(device="cuda").manual_seed(6)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    dx = ops.gemm_a16w4_dgrad(dy, codes, sb, zb, N, K)
    ref = orc.gemm_a16w4(dy.float().cpu().numpy(), codes.cpu().numpy(), sb.float().cpu().numpy(), zb.float().cpu().numpy(),
                         N, K, transpose=True)
    e_max, e_fro = rel_err(dx.cpu(), torch.from_numpy(ref))
    assert e_max < RTOL and e_fro < RTOL, (e_max, e_fro)


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 12288)])
@pytest.mark.parametrize("M", [1, 16, 128, 512, 4096])
def test_a16w4_llama_shapes(ops, a_operand, M, K, N):
    """Benchmark shapes: compare with dequantize (library kernel, itself oracle-checked) + fp32-accumulate matmul."""
    codes, sb, zb = make_w4_layer(ops, N, K, seed=1)
    W = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y = ops.gemm_a16w4_fwd(x, codes, sb, zb, None, N, K)
    ref = (x.float() @ W.float().t())
    e_max, e_fro = rel_err(y, ref)
    assert e_max < RTOL and e_fro < RTOL, ("fwd", e_max, e_fro)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    dx = ops.gemm_a16w4_dgrad(dy, codes, sb, zb, N, K)
    ref = (dy.float() @ W.float())
    e_max, e_fro = rel_err(dx, ref)
    assert e_max < RTOL and e_fro < RTOL, ("dgrad", e_max, e_fro)
    # linearity in the activations: f(2x) == 2 f(x) exactly (power-of-two scaling commutes with rounding)
    y2 = ops.gemm_a16w4_fwd(x * 2, codes, sb, zb, None, N, K)
    assert torch.equal(y2, y * 2)


@pytest.mark.parametrize("M,N,K", [(24, 512, 1024), (64, 320, 2048), (128, 11008, 4096), (200, 4096, 4096), (512, 4096, 11008)])
def test_a16w4_fwd_balanced_plan_vs_oracle(ops, a_operand, monkeypatch, M, N, K):
    """The forward kernel with its (tile, k-block) units dealt out evenly over the SMs: segments that cover part of a
    tile's k range publish their partial sums in the workspace and the last one to finish adds them up in k order.
    Same tolerance as the whole-tile plan, and the same bits on every run (the order of the additions is fixed)."""
    monkeypatch.setenv("LQ_GEMM_BALANCE", "1")
    ops._ws_need.clear()
    codes, sb, zb = make_w4_layer(ops, N, K, seed=M + N)
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    y = ops.gemm_a16w4_fwd(x, codes, sb, zb, bias, N, K)
    W = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16)
    ref = (x.float() @ W.float().t()).to(torch.bfloat16).float() + bias.float()
    e_max, e_fro = rel_err(y, ref)
    assert e_max < RTOL and e_fro < RTOL, (e_max, e_fro)
    assert torch.equal(y, ops.gemm_a16w4_fwd(x, codes, sb, zb, bias, N, K))
    ops._ws_need.clear()


@pytest.mark.parametrize("M,N,K,group", [(300, 384, 1024, 128), (4096, 4096, 4096, 128), (77, 256, 512, 64), (512, 512, 512, 32),
                                         (1000, 2048, 2048, 256)])
def test_a16w4_tmem_and_smem_operand_paths_agree_bitwise(ops, monkeypatch, M, N, K, group):
    """Both placements feed the tensor core the same bf16 weights in the same order: outputs must be identical
    (whole-tile plan for both: the balanced plan's 256-token tile exists for one placement only)."""
    monkeypatch.setenv("LQ_GEMM_BALANCE", "0")
    ops._ws_need.clear()
    codes, sb, zb = make_w4_layer(ops, N, K, seed=7, group=group)
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    out = {}
    for where in ("tmem", "smem"):
        monkeypatch.setenv("LQ_GEMM_A_OPERAND", where)
        out[where] = (ops.gemm_a16w4_fwd(x, codes, sb, zb, None, N, K, group), ops.gemm_a16w4_dgrad(dy, codes, sb, zb, N, K, group))
    assert torch.equal(out["tmem"][0], out["smem"][0])
    assert torch.equal(out["tmem"][1], out["smem"][1])
    W = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16, group)
    e_max, e_fro = rel_err(out["tmem"][0], x.float() @ W.float().t())
    assert e_max < RTOL and e_fro < RTOL


@pytest.mark.parametrize("group", [64, 128, 256])
@pytest.mark.parametrize("M,N,K", [(1, 320, 1024), (5, 4096, 2816), (8, 192, 768), (9, 1088, 2048), (16, 4096, 4096),
                                   (3, 960, 4096), (2, 576, 11008), (8, 4992, 11008), (12, 8960, 2048), (13, 12288, 4096)])
def test_a16w4_decode_sized_forward_all_routes(ops, monkeypatch, M, N, K, group):
    """M <= 16: the streaming row-block kernel (group 128 / 256, at least two groups per warp, tokens staged in shared
    memory; default for M <= 2 and, one CTA per SM, for 9-16 tokens at K = 4096; forced for the rest), the
    one-block-per-CTA row kernel (default otherwise),
    the split-K kernel (group 64, or forced) and the tensor-core kernel (forced) against dequantize + fp32 matmul,
    with bias; ragged row blocks, uneven K slices and more row blocks than persistent CTAs included."""
    if K % group:
        pytest.skip("K must hold whole groups")
    codes, sb, zb = make_w4_layer(ops, N, K, seed=3, group=group)
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    W = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16, group)
    ref = x.float() @ W.float().t() + bias.float()
    for env in ({}, {"LQ_SKINNY_NO_STREAM": "1"}, {"LQ_SKINNY_NO_STREAM16": "1"}, {"LQ_SKINNY_STREAM_ALL": "1"}, {"LQ_SKINNY_SPLIT": "1"},
                {"LQ_GEMM_NO_SKINNY": "1"}):
        for k in ("LQ_SKINNY_SPLIT", "LQ_GEMM_NO_SKINNY", "LQ_SKINNY_NO_STREAM", "LQ_SKINNY_STREAM_ALL", "LQ_SKINNY_NO_STREAM16"):
            monkeypatch.delenv(k, raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        ops._ws_need.clear()            # the plan (and its scratch size) depends on these switches
        y = ops.gemm_a16w4_fwd(x, codes, sb, zb, bias, N, K, group)
        e_max, e_fro = rel_err(y, ref)
        assert e_max < RTOL and e_fro < RTOL, (env, e_max, e_fro)


@pytest.mark.parametrize("M", [1, 2, 8, 16])
def test_a16w4_decode_chain_of_dependent_launches(ops, monkeypatch, M):
    """Decode kernels are launched with programmatic stream serialization: a launch may start (and fetch its weights)
    while its predecessor is still running, but must read its tokens only once the predecessor has finished.  A chain in
    which every launch consumes the previous launch's output, without any synchronisation in between, must give exactly
    the result of the same chain with the early start switched off."""
    K = N = 2048
    layers = [make_w4_layer(ops, N, K, seed=20 + i) for i in range(3)]
    g = torch.Generator(device="cuda").manual_seed(M)
    x0 = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    outs = {}
    for mode in ("pdl", "plain"):
        if mode == "plain":
            monkeypatch.setenv("LQ_SKINNY_NO_PDL", "1")
        else:
            monkeypatch.delenv("LQ_SKINNY_NO_PDL", raising=False)
        bufs = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        x = x0
        with ops.decode_chain():                                # the early start is only ever on inside a decode chain
            for it in range(30):                                # 30 dependent launches, ping-pong buffers
                codes, sb, zb = layers[it % 3]
                y = ops.gemm_a16w4_fwd(x, codes, sb, zb, None, N, K, out=bufs[it % 2])
                x = y
        torch.cuda.synchronize()
        outs[mode] = x.clone()
    assert torch.isfinite(outs["pdl"].float()).all()
    assert torch.equal(outs["pdl"], outs["plain"])


def test_decode_forward_right_after_a_requantize_reads_the_new_weights(ops):
    """Outside a decode chain nothing is fetched early: a decode-sized forward launched directly behind the kernel that
    rewrote its weights (an optimizer step) sees the new codes, with no synchronisation in between."""
    N = K = 2048
    codes, sb, zb = make_w4_layer(ops, N, K, seed=77)
    words = torch.zeros(N * K // 8, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(1, K, device="cuda", generator=g).to(torch.bfloat16)
    delta = (torch.randn(N * K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, has_residual=False)
    torch.cuda.synchronize()
    for _ in range(5):
        ops.a16w4_fold_delta(codes, words, delta, sb, zb, o)          # rewrites the codes ...
        y = ops.gemm_a16w4_fwd(x, codes, sb, zb, None, N, K)          # ... read by the very next launch
        torch.cuda.synchronize()
        assert torch.equal(y, ops.gemm_a16w4_fwd(x, codes, sb, zb, None, N, K))
        o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH, has_residual=True)


def _a8_inputs(M, N, K, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    out_ch = rng.choice(K, max(1, K // 100), replace=False)
    x[:, out_ch] *= 20.0
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    w_scale = (np.abs(w).max(axis=1) / 127.0).astype(np.float32)
    w8 = np.clip(np.rint(w / w_scale[:, None]), -128, 127).astype(np.int8)
    bias = orc.bf16_round((rng.standard_normal(N) * 0.1).astype(np.float32))
    return x, w8, w_scale, bias


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 256, 256), (37, 192, 384), (130, 128, 1024), (300, 320, 512)])
def test_a8w8_small_vs_oracle(ops, M, N, K):
    x, w8, w_scale, bias = _a8_inputs(M, N, K, seed=M)
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    x8, a_scale = ops.act_quant_per_token(xb)
    y, acc = ops.gemm_a8w8(x8, torch.from_numpy(w8).cuda(), a_scale, torch.from_numpy(w_scale).cuda(), 1.0,
                           torch.from_numpy(bias).cuda().to(torch.bfloat16), want_acc=True)
    acc_o = orc.gemm_i8_acc(x8.cpu().numpy(), w8)
    assert np.array_equal(acc.cpu().numpy(), acc_o)                       # int32 accumulators: bit-exact
    y_o = orc.gemm_i8_epilogue_fused(acc_o, a_scale.cpu().numpy(), w_scale, bias)
    assert np.array_equal(y.float().cpu().numpy(), y_o)                   # epilogue restated op for op
    # the torch_int call form: alpha only
    y2 = ops.gemm_a8w8(x8, torch.from_numpy(w8).cuda(), None, None, 0.0123, torch.from_numpy(bias).cuda().to(torch.bfloat16))
    assert np.array_equal(y2.float().cpu().numpy(), orc.gemm_i8_epilogue_torch_int(acc_o, 0.0123, bias))
    # against the floating-point product it approximates
    ref = x @ (w8.astype(np.float32) * w_scale[:, None]).T + bias
    e_max, e_fro = rel_err(y.float().cpu(), torch.from_numpy(ref))
    assert e_fro < 6e-2, (e_max, e_fro)     # int8 quantization error of the product itself (outlier channels x20)


@pytest.mark.parametrize("K,N", [(2048, 2048), (2048, 8192), (8192, 2048)])
@pytest.mark.parametrize("M", [2048, 16384])
def test_a8w8_opt_shapes(ops, M, K, N):
    g = torch.Generator(device="cuda").manual_seed(K + N)
    x8 = torch.randint(-128, 128, (M, K), device="cuda", generator=g, dtype=torch.int8)
    w8 = torch.randint(-128, 128, (N, K), device="cuda", generator=g, dtype=torch.int8)
    y, acc = ops.gemm_a8w8(x8, w8, None, None, 1e-4, None, want_acc=True)
    # exact integer reference on the device: fp64 matmul of int8 values is exact (|acc| < 2^53)
    mrows = min(M, 1024)
    ref = (x8[:mrows].double() @ w8.double().t()).to(torch.int64)
    assert torch.equal(acc[:mrows].to(torch.int64), ref)
    # checksum of checksums over the full output: sum_n acc[m, n] == x8[m, :] · sum_n w8[n, :]
    colsum = w8.to(torch.int64).sum(0)
    want = (x8.to(torch.int64) * colsum[None, :]).sum(1)
    assert torch.equal(acc.to(torch.int64).sum(1), want)


@pytest.mark.parametrize("K,N", [(2048, 2048), (2048, 8192), (8192, 2048)])
def test_a8w8_full_forward_opt_shapes_m2048(ops, K, N):
    """The whole A8W8 forward at benchmark size (M = 4x512 tokens, OPT-1.3B shapes): activations ~N(0,1) with 1 % of the
    channels scaled x20, per-token activation quantizer on the GPU, int8 GEMM with per-token and per-channel scales and
    bias in its epilogue.  Quantized activations and scales against the oracle bit for bit; the bf16 output against the
    oracle's epilogue applied to exact integer accumulators (computed on the device in fp64), bit for bit."""
    M = 2048
    x, w8, w_scale, bias = _a8_inputs(M, N, K, seed=K + N)
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    x8, a_scale = ops.act_quant_per_token(xb)
    q_o, s_o = orc.act_quant_per_token(xb.float().cpu().numpy(), math_bf16=True)
    assert np.array_equal(x8.cpu().numpy(), q_o) and np.array_equal(a_scale.cpu().numpy(), s_o)
    w8d = torch.from_numpy(w8).cuda()
    y = ops.gemm_a8w8(x8, w8d, a_scale, torch.from_numpy(w_scale).cuda(), 1.0, torch.from_numpy(bias).cuda().to(torch.bfloat16))
    acc = (x8.double() @ w8d.double().t()).to(torch.int64).cpu().numpy().astype(np.int32)      # exact: |acc| < 2^31
    y_o = orc.gemm_i8_epilogue_fused(acc, s_o, w_scale, bias)
    assert np.array_equal(y.float().cpu().numpy(), y_o)
    ref = xb.float().cpu().numpy() @ (w8.astype(np.float32) * w_scale[:, None]).T + bias
    _, e_fro = rel_err(y.float().cpu(), torch.from_numpy(ref))
    assert e_fro < 6e-2, e_fro              # the int8 quantization error of the product itself


@pytest.mark.parametrize("M,N,K", [(2048, 2048, 2048), (300, 320, 192), (64, 128, 64), (4096, 1024, 8192), (1000, 136, 264)])
def test_wgrad_gemm_vs_fp32_matmul(ops, M, N, K):
    """dw (+)= dy^T x on tcgen05 with both operands MN-major: against an fp32 matmul, written and accumulated (one
    rounding of fp32(dw) + product, like a GEMM with beta = 1), on full tiles and ragged edges."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    prod = dy.float().t() @ x.float()
    dw = ops.gemm_wgrad(dy, x)
    e_max, e_fro = rel_err(dw, prod)
    assert e_max < RTOL and e_fro < RTOL, (e_max, e_fro)
    old = (torch.randn(N, K, device="cuda", generator=g) * prod.abs().mean()).to(torch.bfloat16)
    acc = old.clone()
    ops.gemm_wgrad(dy, x, acc, accumulate=True)
    want = (old.float() + prod).to(torch.bfloat16)
    e_max, e_fro = rel_err(acc, want.float())
    assert e_max < RTOL and e_fro < RTOL, (e_max, e_fro)
    assert float((acc == want).float().mean()) > 0.9                 # same single rounding: only the fp32 sum order differs
    # linearity: doubling dy doubles the product exactly
    assert torch.equal(ops.gemm_wgrad(dy * 2, x), dw * 2)


def test_mma_issue_rate_probe_runs_and_rejects_bad_arguments():
    """`lq_mma_issue_rate` (the tensor-core ceiling the GEMM rooflines quote): a short run returns a plausible cycle
    count per 128 x 256 MMA (the ideal is 128 cycles for either kind), and argument errors come back as LQ_EINVAL
    without a launch."""
    import ctypes as C
    from latentq_llm_b200 import _lib
    lib = _lib.lib
    torch.zeros(1, device="cuda")
    for kind, ta in ((_lib.GEMM_A16W4_FWD, 0), (_lib.GEMM_A16W4_FWD, 1), (_lib.GEMM_A8W8, 0)):
        cyc = C.c_ulonglong(0)
        assert lib.lq_mma_issue_rate(kind, ta, 256, 1, 1024, 4, C.byref(cyc), None) == 0
        assert 100.0 <= cyc.value / 1024 <= 400.0, (kind, ta, cyc.value / 1024)
    cyc = C.c_ulonglong(0)
    assert lib.lq_mma_issue_rate(_lib.GEMM_A16W4_FWD, 0, 250, 1, 1024, 4, C.byref(cyc), None) == _lib.LQ_EINVAL     # N not a multiple of 16
    assert lib.lq_mma_issue_rate(_lib.GEMM_A16W4_FWD, 0, 256, 2, 1024, 4, C.byref(cyc), None) == _lib.LQ_EINVAL     # accumulators beyond 256 columns
    assert lib.lq_mma_issue_rate(_lib.GEMM_A8W8, 1, 256, 1, 1024, 4, C.byref(cyc), None) == _lib.LQ_EINVAL          # int8 has no tensor-memory A here


@pytest.mark.parametrize("K", [4096, 11008])
@pytest.mark.parametrize("M,N,force_stream", [(1, 4096, True), (2, 12288, True), (1, 1088, True), (12, 4160, True),
                                              (5, 4096, False), (16, 12288, False), (9, 1088, False), (3, 4160, False)])
def test_a16w4_decode_kernels_written_out_loop_equals_general_loop(ops, monkeypatch, M, N, force_stream, K):
    """K = 4096 with groups of 128 runs the decode kernels' written-out loops (four chunks per warp, group parameters
    as 8-byte loads, constant offsets): the streaming kernel (one or two tokens, or forced) and the row-block kernel.
    Same operations in the same order as the general loops: identical bits, with bias, for more and for fewer row
    blocks than persistent CTAs, one and two token groups; the fused gate|up + silu epilogue included.  K = 11008 (eleven
    chunks per warp, nine in the last one) has written-out loops of its own."""
    codes, sb, zb = make_w4_layer(ops, N, K, seed=11)
    g = torch.Generator(device="cuda").manual_seed(N + M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    if force_stream:
        monkeypatch.setenv("LQ_SKINNY_STREAM_ALL", "1")         # (M = 12 takes the streaming kernel only when forced)
    out = {}
    for mode in ("written_out", "general"):
        if mode == "general":
            monkeypatch.setenv("LQ_SKINNY_NO_NC4", "1")
        else:
            monkeypatch.delenv("LQ_SKINNY_NO_NC4", raising=False)
        ops._ws_need.clear()
        y = ops.gemm_a16w4_fwd(x, codes, sb, zb, bias, N, K)
        act = ops.gemm_a16w4_fwd_silu(x, codes, sb, zb, N // 2, K, hf_rounding=1) if N % 16 == 0 else None
        out[mode] = (y, act)
    assert torch.equal(out["written_out"][0], out["general"][0])
    if out["general"][1] is not None:
        assert torch.equal(out["written_out"][1], out["general"][1])
    W = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16)
    e_max, e_fro = rel_err(out["written_out"][0], x.float() @ W.float().t() + bias.float())
    assert e_max < RTOL and e_fro < RTOL
    ops._ws_need.clear()


@pytest.mark.parametrize("M,N,K,force", [(3072, 4096, 4096, False), (3100, 11008, 4096, False), (4096, 4096, 11008, False),
                                         (300, 512, 1024, True), (257, 192, 512, True)])
def test_a16w4_dgrad_through_transposed_copy(ops, monkeypatch, M, N, K, force):
    """From 3072 tokens on the grad-input GEMM transposes the packed weight (and lays its group parameters out per
    contraction element) into the workspace and runs the forward kernel on the copy.  Against dequantize + fp32 matmul
    with the GEMM tolerance, and against the kernel that reads the weight as stored; ragged token tiles, row counts that
    are not multiples of the 128-row tile, and small shapes with the route forced."""
    codes, sb, zb = make_w4_layer(ops, N, K, seed=5)
    g = torch.Generator(device="cuda").manual_seed(M + K)
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    W = ops.a16w4_dequant(codes, sb, zb, (N, K), torch.bfloat16)
    ref = dy.float() @ W.float()
    out = {}
    for mode in ("copy", "stored"):
        monkeypatch.setenv("LQ_GEMM_DGRAD_TRANSPOSE", "0" if mode == "stored" else ("1" if force else ""))
        if mode == "copy" and not force:
            monkeypatch.delenv("LQ_GEMM_DGRAD_TRANSPOSE", raising=False)
        ops._ws_need.clear()
        out[mode] = ops.gemm_a16w4_dgrad(dy, codes, sb, zb, N, K)
        e_max, e_fro = rel_err(out[mode], ref)
        assert e_max < RTOL and e_fro < RTOL, (mode, e_max, e_fro)
    # both kernels feed the tensor core the same bf16 weights, k-block after k-block: where neither splits the contraction
    # (the large shapes) the bits agree
    if not force:
        assert torch.equal(out["copy"], out["stored"])
    ops._ws_need.clear()


@pytest.mark.parametrize("hf", [1, 0])
@pytest.mark.parametrize("with_delta", [True, False])
@pytest.mark.parametrize("M,N", [(1, 12288), (2, 12288), (1, 22016), (2, 22016), (2, 9600)])
def test_a16w4_decode_forward_with_residual_add_and_rmsnorm_in_the_launch(ops, M, N, with_delta, hf):
    """One or two tokens at K = 4096: the streaming decode kernel computes RMSNorm(h + delta) * gamma while it stages
    its tokens.  The new residual stream and the projection are bit for bit those of `add_rmsnorm` followed by the
    GEMM (plain and gate|up + silu), with and without a delta, in both rounding modes of the norm; other shapes
    answer LQ_EUNSUPPORTED (None) and write nothing."""
    K = 4096
    codes, sb, zb = make_w4_layer(ops, N, K, seed=23)
    g = torch.Generator(device="cuda").manual_seed(N + M + hf)
    h = (torch.randn(M, K, device="cuda", generator=g) * 2).to(torch.bfloat16)
    delta = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16) if with_delta else None
    gamma = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16)
    eps = 1e-5
    for silu in (False, True):
        if silu and N % 16:
            continue
        h_ref = h.clone()
        xn = ops.add_rmsnorm(h_ref, delta, gamma, eps, hf_rounding=hf)          # h_ref += delta in place
        if silu:
            want = ops.gemm_a16w4_fwd_silu(xn, codes, sb, zb, N // 2, K, hf_rounding=hf)
        else:
            want = ops.gemm_a16w4_fwd(xn, codes, sb, zb, None, N, K)
        h_in, h_out = h.clone(), torch.full_like(h, 7.0)
        got = ops.gemm_a16w4_fwd_rmsnorm(h_in, delta, gamma, eps, h_out, codes, sb, zb, N, K, silu_pair=silu, hf_rounding=hf)
        assert got is not None
        assert torch.equal(got, want)
        assert torch.equal(h_in, h)                                              # the input stream is left alone
        if with_delta:
            assert torch.equal(h_out, h_ref)
        else:
            assert torch.equal(h_out, torch.full_like(h, 7.0))                   # nothing to add: nothing written


def test_a16w4_rmsnorm_forward_refuses_shapes_without_a_fused_kernel(ops):
    for M, N, K in [(3, 12288, 4096), (1, 12288, 2048), (16, 12288, 4096), (1, 12288, 11008), (1, 4096, 4096)]:   # the last: one row block per CTA
        codes, sb, zb = make_w4_layer(ops, N, K, seed=3)
        h = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        gamma = torch.ones(K, device="cuda", dtype=torch.bfloat16)
        y = torch.full((M, N), 3.0, device="cuda", dtype=torch.bfloat16)
        assert ops.gemm_a16w4_fwd_rmsnorm(h, None, gamma, 1e-5, None, codes, sb, zb, N, K, out=y) is None
        assert torch.equal(y, torch.full_like(y, 3.0))


@pytest.mark.parametrize("hf", [1, 0])
@pytest.mark.parametrize("M,Hq,Hkv,hd,K,with_norm", [(1, 32, 32, 128, 4096, True), (2, 32, 8, 128, 4096, True), (1, 8, 8, 128, 4096, False),
                                                     (16, 32, 32, 128, 4096, False), (5, 8, 2, 64, 2048, False), (2, 4, 4, 64, 256, False),
                                                     (9, 8, 4, 128, 11008, False)])
def test_a16w4_qkv_projection_with_rope_and_cache_write_as_its_epilogue(ops, M, Hq, Hkv, hd, K, with_norm, hf):
    """Up to 16 tokens: the q|k|v projection pairs rows i and i + hd/2 of a head in one MMA block and finishes with the
    rotary embedding and the KV-cache write.  The projection buffer (q rotated, k and v as projected) and both caches
    are bit for bit those of the GEMM followed by `rope_kv_store`, for full and grouped KV heads, head sizes 64 and
    128, both rounding modes, a position beyond the cache (nothing written), and with the residual add + RMSNorm in the
    same launch (one or two tokens, K = 4096)."""
    N, max_len = (Hq + 2 * Hkv) * hd, 80
    codes, sb, zb = make_w4_layer(ops, N, K, seed=29)
    g = torch.Generator(device="cuda").manual_seed(N + M + hf)
    h = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    delta = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16)
    pos = torch.randint(0, max_len, (M,), device="cuda", generator=g)
    if M > 1:
        pos[M - 1] = max_len + 3                     # beyond the cache: the caches stay untouched for that token
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).cuda()
    kc = (torch.randn(M, Hkv, max_len, hd, device="cuda", generator=g)).to(torch.bfloat16)
    vc = (torch.randn(M, Hkv, max_len, hd, device="cuda", generator=g)).to(torch.bfloat16)
    eps = 1e-5
    # two launches (three with the norm)
    h_ref, kc_ref, vc_ref = h.clone(), kc.clone(), vc.clone()
    x = ops.add_rmsnorm(h_ref, delta, gamma, eps, hf_rounding=hf) if with_norm else h
    want = ops.gemm_a16w4_fwd(x, codes, sb, zb, None, N, K)
    ops.rope_kv_store(want, pos, inv_freq, kc_ref, vc_ref, Hq, Hkv, hd, hf_rounding=hf)
    # one launch
    kc_got, vc_got, h_out = kc.clone(), vc.clone(), torch.zeros_like(h)
    norm = (h.clone(), delta, gamma, eps, h_out) if with_norm else None
    got = ops.gemm_a16w4_fwd_qkv_rope(None if with_norm else h, codes, sb, zb, pos, inv_freq, kc_got, vc_got, Hq, Hkv, hd, K,
                                      hf_rounding=hf, norm=norm)
    assert got is not None
    assert torch.equal(got, want)
    assert torch.equal(kc_got, kc_ref) and torch.equal(vc_got, vc_ref)
    assert not torch.equal(kc_got, kc)               # the caches did receive the in-range tokens
    if with_norm:
        assert torch.equal(h_out, h_ref)


def test_a16w4_qkv_rope_projection_refuses_what_it_does_not_serve(ops):
    Hq = Hkv = 4
    for M, hd, K in [(17, 128, 4096), (2, 24, 1024)]:
        codes, sb, zb = make_w4_layer(ops, 64, K, seed=3)            # refused before anything is read
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        pos = torch.zeros(M, dtype=torch.long, device="cuda")
        inv_freq = torch.ones(hd // 2, device="cuda")
        kc = torch.zeros(M, Hkv, 8, hd, dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        assert ops.gemm_a16w4_fwd_qkv_rope(x, codes, sb, zb, pos, inv_freq, kc, vc, Hq, Hkv, hd, K) is None
        assert not kc.any() and not vc.any()
