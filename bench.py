#!/usr/bin/env python
"""Benchmark of the quantized-weight hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the A16W4 hot path over one batch of synthetic activations: the quantized
linear forward (y = x·deq(Wq)^T) and grad-input (dx = dy·deq(Wq)) for the four Llama-2-7B linear shapes
at M = 4096 tokens (8 GEMMs = 16 kernel launches: each grad-input of this size first writes a transposed copy
of the packed weight and its group parameters with two small kernels, inside the timed region).  Rank r of N runs an independent replica of the same work on its
own GPU ("replicas only": the kernels have no exchange step), the timed region is bracketed by a
barrier + synchronize, timed with CUDA events on the launching stream, and the maximum over ranks is
reported.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA_SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 12288)]   # (K, N)
M_TOKENS = 4096
GROUP = 128
METRIC = "a16w4_gemm_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "A16W4 dequant-GEMM fwd+grad-input, Llama-2-7B linear shapes (K,N) in {(4096,4096),(4096,11008),(11008,4096),(4096,12288)}, M=4096, group 128"


# dram__bytes_read.sum + dram__bytes_write.sum per k_gemm launch from an ncu capture of the (K,N)=(4096,11008),
# M=4096 launches (a tensor-bound kernel: the figure shows there are no re-reads)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 132.6e6
NCU_TRAFFIC_NOTE = ("ncu capture of the (K,N)=(4096,11008), M=4096 launches: forward 116.0 MB, grad-input 149.3 MB, mean 132.6 MB "
                    "per launch against 146.8 MB algorithmic bytes of that shape")


def step_flops(m=M_TOKENS):
    return sum(2 * 2.0 * m * n * k for (k, n) in LLAMA_SHAPES)   # fwd + dgrad


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "src": "fallback"}


def roofline_entry(per_gpu_tflops, pk, clocks):
    """Tensor roofline of the headline kernel.  The denominator is the burst cuBLAS figure when the SM clock sampled
    during the timed region stayed near its maximum (the conditions the burst figure was taken under), else the
    sustained one; both fractions are given."""
    sm, mx = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    burst = bool(sm and mx and sm >= 0.9 * mx)
    peak = pk["bf16"] if burst else pk["bf16_sustained"]
    return {"bound": "tensor", "achieved": round(per_gpu_tflops, 2), "peak": peak, "unit": "TFLOP/s",
            "frac": round(per_gpu_tflops / peak, 4), "frac_of_burst": round(per_gpu_tflops / pk["bf16"], 4),
            "frac_of_sustained": round(per_gpu_tflops / pk["bf16_sustained"], 4),
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "traffic_note": NCU_TRAFFIC_NOTE,
            "peak_source": pk["src"] + (" (burst bf16 cuBLAS figure: SM clock during the timed region near its maximum)" if burst else
                                        " (sustained bf16 cuBLAS figure: SM clock during the timed region well below its maximum)"),
            "kernel": "k_gemm<A16W4 fwd/dgrad, 256 tokens>", "algorithmic": "2*M*N*K flops per launch"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.strip().split(",") for r in open(self.f.name) if r.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons, pw = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); pw.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for nm, v in zip(names, r[3:7]):
                if v.strip().lower().startswith("active"):
                    reasons.add(nm)
        # samples under load = upper half of the power readings
        if sm:
            thr = statistics.median(pw)
            load = [s for s, w in zip(sm, pw) if w >= thr] or sm
            return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                    "power_w_max": max(pw)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}


# ------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------
def build_layers(torch, ops, seed=1234):
    """Synthetic Llama-2-7B-shaped layers: W ~ N(0, 0.02) -> group-128 asymmetric int4 (nibble-pair layout)."""
    layers = []
    g = torch.Generator(device="cuda").manual_seed(seed)
    for (k, n) in LLAMA_SHAPES:
        w = (torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        s, z = ops.find_qparams(w, GROUP, 15, False)
        sb, zb = s.to(torch.bfloat16), z.to(torch.bfloat16)
        codes, _ = ops.a16w4_requant(w, sb, zb, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16), group=GROUP)
        x = torch.randn(M_TOKENS, k, device="cuda", generator=g).to(torch.bfloat16)
        dy = torch.randn(M_TOKENS, n, device="cuda", generator=g).to(torch.bfloat16)
        layers.append(dict(K=k, N=n, codes=codes, s=sb, z=zb, x=x, dy=dy,
                           y=torch.empty(M_TOKENS, n, device="cuda", dtype=torch.bfloat16),
                           dx=torch.empty(M_TOKENS, k, device="cuda", dtype=torch.bfloat16)))
        del w
    return layers


def launches_per_layer(m=M_TOKENS):
    """Kernel launches of one forward + one grad-input: from 3072 tokens on the grad-input is three launches
    (weight transpose, group-parameter transpose, GEMM) unless the route is switched off."""
    transposed = (m >= 3072 and os.environ.get("LQ_GEMM_DGRAD_TRANSPOSE") != "0" and "LQ_GEMM_A_OPERAND" not in os.environ)
    return 4 if transposed else 2


def run_step(ops, layers):
    for L in layers:
        ops.gemm_a16w4_fwd(L["x"], L["codes"], L["s"], L["z"], None, L["N"], L["K"], out=L["y"])
        ops.gemm_a16w4_dgrad(L["dy"], L["codes"], L["s"], L["z"], L["N"], L["K"], out=L["dx"])
    return launches_per_layer() * len(layers)


def timed(torch, fn, steps, barrier):
    barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launches = 0
    for _ in range(steps):
        launches += fn()
    e1.record()
    torch.cuda.synchronize(); barrier()
    return e0.elapsed_time(e1), launches


def extra_measurements(torch, ops, pk, only=None, numel=1 << 30):
    """Secondary figures of the same hot path (not the headline): requantize GB/s, int8 GEMM TOP/s, decode-size GEMM.
    `only` restricts to one family ("requant", "a8w8", "decode") for profiling runs."""
    out = {}

    def tm(fn, reps=5, warm=2, graph=False):
        """Mean device time of one call in ms.  graph=True: `reps` calls are captured into one CUDA graph and the graph
        is replayed (best of 3), so that host time between short launches (Python, output allocation) is not in the
        figure; falls back to eager timing if the call cannot be captured."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if graph:
            try:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    for _ in range(reps):
                        fn()
                gr.replay(); torch.cuda.synchronize()
                best = float("inf")
                for _ in range(3):
                    e0.record(); gr.replay(); e1.record(); torch.cuda.synchronize()
                    best = min(best, e0.elapsed_time(e1) / reps)
                del gr
                return best
            except Exception:
                torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    g = torch.Generator(device="cuda").manual_seed(7)
    if only in (None, "requant"):
        _requant_part(torch, ops, pk, out, tm, g, numel)
    if only in (None, "sweep"):
        _sweep_part(torch, ops, pk, out, tm, g)
        torch.cuda.empty_cache()
    if only in (None, "stream"):
        _stream_part(torch, ops, pk, out, tm, g)
    if only in (None, "a8w8"):
        _a8w8_part(torch, ops, out, tm, g)
    if only in (None, "decode"):
        _decode_part(torch, ops, pk, out, tm)
    if only == "mma_probe":
        out["mma_issue_rate"] = mma_probe_sweep(torch)
    if only in (None, "wgrad"):
        _wgrad_part(torch, ops, pk, out, tm, g)
    if only == "decode_step":
        _decode_step_part(torch, out, layers=DECODE_STEP_ARGS["layers"], batch=DECODE_STEP_ARGS["batch"])
    return out


DECODE_STEP_ARGS = {"layers": 4, "batch": 1}


def _decode_step_part(torch, out, layers=4, batch=1, prompt_len=512):
    """One decode step of the Llama-2-7B architecture (first `layers` layers) through the fused kernel chain, run eagerly
    between cudaProfilerStart / cudaProfilerStop (for `ncu --profile-from-start off`), and timed as a graph replay."""
    from latentq_llm_b200 import finetune as ft
    from latentq_llm_b200.generate import FusedLlamaGreedyDecoder
    model = ft.build_model("llama-2-7b", "cuda", seed=1, layers=layers)
    ft.quantize_decoder(model, lbit=0, gbit=16)
    model.eval()
    prompt = torch.randint(0, 32000, (batch, prompt_len), device="cuda")
    dec = FusedLlamaGreedyDecoder(model, batch=batch, max_len=prompt_len + 72)
    dec.generate(prompt, 4)                      # capture + warm-up
    dec.generate(prompt, 2, use_graph=False)
    torch.cuda.synchronize()
    with torch.no_grad():
        torch.cuda.profiler.start()
        dec._step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(32):
        dec.graph.replay()
    e1.record(); torch.cuda.synchronize()
    out["decode_step"] = {"layers": layers, "batch": batch, "ms_per_step_graph": round(e0.elapsed_time(e1) / 32, 4)}


def _requant_part(torch, ops, pk, out, tm, g, numel):
    # requantize: fold a bf16 update into codes+residual (codes 0.5 + residual 0.5 read and written, delta 2 B read)
    codes = torch.randint(-128, 128, (numel // 2,), device="cuda", generator=g, dtype=torch.int8)
    words = torch.zeros(numel // 8, dtype=torch.int32, device="cuda")
    delta = (torch.randn(numel, device="cuda", generator=g, dtype=torch.bfloat16) * 1e-4)
    s = torch.full((numel // GROUP,), 0.008, device="cuda", dtype=torch.bfloat16)
    z = torch.full((numel // GROUP,), 8.0, device="cuda", dtype=torch.bfloat16)
    bytes_per = 4.0 + 4.0 / GROUP
    for name, kw in (("threefold_hash", dict(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH)),
                     ("threefold_philox", dict(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_PHILOX)),
                     ("uniform16_philox", dict(codec=ops.CODEC_UNIFORM16, dither=ops.DITHER_PHILOX))):
        o = ops.make_opts(seed=1, step=1, param_id=0, **kw)
        ms = tm(lambda: ops.a16w4_fold_delta(codes, words, delta, s, z, o))
        gbs = bytes_per * numel / ms / 1e6
        out["requant_" + name] = {"GB/s": round(gbs, 1), "frac_hbm": round(gbs / pk["hbm_gbs"], 3), "ms": round(ms, 3), "numel": numel}
        import ctypes
        from latentq_llm_b200 import _lib
        cnt = ctypes.c_ulonglong(0)
        _lib.lib.lq_fold_fallback_words(1, ctypes.byref(cnt))
        out["requant_" + name]["generic_fallback_words"] = cnt.value
    # same for int8 codes with one scale per weight row of 4096 (A8W8): codes 1 B + residual 0.5 B read and written, delta 2 B
    n8 = numel // 2
    codes8 = torch.randint(-100, 100, (n8 // 4096, 4096), device="cuda", generator=g, dtype=torch.int8)
    qs8 = torch.full((n8 // 4096,), 0.0006, device="cuda", dtype=torch.bfloat16)
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH)
    ms = tm(lambda: ops.a8w8_fold_delta(codes8, words[:n8 // 8], delta[:n8], qs8, o))
    gbs = (5.0 + 2.0 / 4096) * n8 / ms / 1e6
    cnt = ctypes.c_ulonglong(0)
    _lib.lib.lq_fold_fallback_words(1, ctypes.byref(cnt))
    out["requant_a8w8_threefold_hash"] = {"GB/s": round(gbs, 1), "frac_hbm": round(gbs / pk["hbm_gbs"], 3), "ms": round(ms, 3),
                                          "numel": n8, "generic_fallback_words": cnt.value}
    del delta, codes8, qs8
    # fused optimizer step (8-bit state decode + Adam + state re-encode + requantize in one pass): codes and residual
    # read and written (2 x 1 B), bf16 gradient read (2 B), two uint8 states read and written (4 B) = 8 B per weight
    n2 = numel // 4
    grad = (torch.randn(n2, device="cuda", generator=g, dtype=torch.bfloat16) * 1e-3)
    st1 = torch.zeros(n2, dtype=torch.uint8, device="cuda"); st2 = torch.zeros_like(st1)
    blk = [torch.full((n2 // 2048,), 1e-10, dtype=torch.float32, device="cuda") if i % 2 == 0 else
           torch.zeros(n2 // 2048, dtype=torch.float32, device="cuda") for i in range(4)]
    hyper = ops.make_adam_hyper(0.9, 0.95, 1e-8, 1e-3)
    o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=ops.DITHER_HASH)
    ms = tm(lambda: ops.adam_a16w4_step(codes[:n2 // 2], words[:n2 // 8], grad, s[:n2 // GROUP], z[:n2 // GROUP],
                                        st1, blk[0], blk[1], st2, blk[2], blk[3], hyper, o))
    gbs = (8.0 + 4.0 / GROUP + 16.0 / 2048) * n2 / ms / 1e6
    out["adam_a16w4_fused"] = {"GB/s": round(gbs, 1), "frac_hbm": round(gbs / pk["hbm_gbs"], 3), "ms": round(ms, 3), "numel": n2}
    del codes, words, s, z, grad, st1, st2


def _sweep_part(torch, ops, pk, out, tm, g):
    """fold_delta GB/s over the weight counts of the requantize sweep (1e8 .. 7e9 weights, the last one beyond 2^32)."""
    sizes = [int(x) // 2048 * 2048 for x in (1e8, 3e8, 1e9, 3e9, 7e9)]
    nmax = sizes[-1]
    codes = torch.randint(-128, 128, (nmax // 2,), device="cuda", generator=g, dtype=torch.int8)
    words = torch.zeros(nmax // 8, dtype=torch.int32, device="cuda")
    delta = torch.empty(nmax, device="cuda", dtype=torch.bfloat16)
    for a in range(0, nmax, 1 << 30):
        b = min(nmax, a + (1 << 30))
        delta[a:b] = torch.randn(b - a, device="cuda", generator=g, dtype=torch.bfloat16) * 1e-4
    s = torch.full((nmax // GROUP,), 0.008, device="cuda", dtype=torch.bfloat16)
    z = torch.full((nmax // GROUP,), 8.0, device="cuda", dtype=torch.bfloat16)
    rows = []
    for n in sizes:
        row = {"numel": n}
        for name, dith in (("hash", ops.DITHER_HASH), ("philox", ops.DITHER_PHILOX)):
            o = ops.make_opts(codec=ops.CODEC_THREEFOLD, dither=dith, seed=1, step=1, param_id=0)
            ms = tm(lambda: ops.a16w4_fold_delta(codes[:n // 2], words[:n // 8], delta[:n], s[:n // GROUP], z[:n // GROUP], o))
            gbs = (4.0 + 4.0 / GROUP) * n / ms / 1e6
            row[name] = {"GB/s": round(gbs, 1), "frac_hbm": round(gbs / pk["hbm_gbs"], 3), "ms": round(ms, 3)}
        rows.append(row)
    out["requant_sweep_threefold"] = rows
    del codes, words, delta, s, z


def _stream_part(torch, ops, pk, out, tm, g, numel=1 << 28):
    """The other HBM-streaming entry points of the path, GB/s over their algorithmic bytes (inputs + outputs)."""
    def rec(name, nbytes, fn):
        ms = tm(fn, reps=20, warm=2, graph=True)          # 20 calls per graph replay: device time only
        out["stream_" + name] = {"GB/s": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3), "ms": round(ms, 3)}
    n = numel
    w = (torch.randn(n, device="cuda", generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    s, z = ops.find_qparams(w, GROUP, 15, False)
    sb, zb = s.to(torch.bfloat16), z.to(torch.bfloat16)
    rec("find_qparams_bf16", 2.0 * n + 8.0 * n / GROUP, lambda: ops.find_qparams(w, GROUP, 15, False))
    codes, _ = ops.a16w4_requant(w, sb, zb, ops.make_opts(codec=ops.CODEC_NONE, math_dtype=torch.bfloat16))
    rec("a16w4_dequant_bf16", 0.5 * n + 2.0 * n + 4.0 * n / GROUP, lambda: ops.a16w4_dequant(codes, sb, zb, (n // 4096, 4096), torch.bfloat16))
    u8 = torch.randint(0, 16, (n,), device="cuda", generator=g, dtype=torch.uint8)
    rec("pack_nibbles", 1.5 * n, lambda: ops.pack_nibbles(u8))
    rec("unpack_nibbles", 1.5 * n, lambda: ops.unpack_nibbles(codes))
    del u8, codes
    x = torch.randn(n, device="cuda", generator=g, dtype=torch.float32)
    rec("opt8_quant", 5.0 * n + 8.0 * n / 2048, lambda: ops.opt8_quant(x, 2048))
    q, sc, tmx = ops.opt8_quant(x, 2048)
    rec("opt8_dequant", 5.0 * n + 8.0 * n / 2048, lambda: ops.opt8_dequant(q, 2048, sc, tmx))
    del x, q
    xa = w.view(-1, 4096)
    rec("act_quant_per_token", 3.0 * n + 4.0 * n / 4096, lambda: ops.act_quant_per_token(xa))
    del w, xa


def mma_peaks(torch):
    """Measured tensor-core ceilings from the library's tcgen05.mma issue-rate microbenchmark (one CTA per SM, operands
    resident in shared memory / tensor memory, ~50 ms per run): int8 TOP/s and bf16 TFLOP/s."""
    import ctypes
    from latentq_llm_b200 import _lib
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    res = {}
    for name, kind, ta, kk in (("int8_tops_measured", _lib.GEMM_A8W8, 0, 32), ("bf16_tflops_mma_smem_a", 0, 0, 16),
                               ("bf16_tflops_mma_tmem_a", 0, 1, 16)):
        n_mma = 1 << 19
        _lib.lib.lq_mma_issue_rate(kind, ta, 256, 1, 4096, sms, None, None)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = _lib.lib.lq_mma_issue_rate(kind, ta, 256, 1, n_mma, sms, None, None)
        e1.record(); torch.cuda.synchronize()
        assert rc == 0
        res[name] = round(2.0 * 128 * 256 * kk * n_mma * sms / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1)
    res["note"] = "128x256 MMAs, one accumulator, all SMs, about 50 ms per figure"
    return res


def mma_probe_sweep(torch):
    """Cycles per tcgen05.mma and T(FL)OP/s over token-tile widths and numbers of independent accumulators."""
    import ctypes
    from latentq_llm_b200 import _lib
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows = []
    for name, kind, ta, kk in (("bf16_smem_a", 0, 0, 16), ("bf16_tmem_a", 0, 1, 16), ("int8_smem_a", _lib.GEMM_A8W8, 0, 32)):
        for n in (32, 64, 128, 256):
            for n_acc in (1, 2, 4, 8):
                if n_acc * n > 256:
                    continue
                cyc = ctypes.c_ulonglong(0)
                assert _lib.lib.lq_mma_issue_rate(kind, ta, n, n_acc, 8192, sms, ctypes.byref(cyc), None) == 0
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                _lib.lib.lq_mma_issue_rate(kind, ta, n, n_acc, 8192, sms, None, None)
                e1.record(); torch.cuda.synchronize()
                rows.append({"kind": name, "N": n, "accumulators": n_acc, "cycles_per_mma": round(cyc.value / 8192, 1),
                             "T(FL)OP/s": round(2.0 * 128 * n * kk * 8192 * sms / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1)})
    return rows


def _a8w8_part(torch, ops, out, tm, g):
    # int8 GEMM on the OPT-1.3B shapes at M = 4x512 and 32x512 tokens, the whole A8W8 forward: per-token activation
    # quantizer, then the GEMM with per-token and per-channel scales and bias in its epilogue (bf16 out).  Activations
    # ~N(0,1) with 1 % of the channels scaled x20.  The denominator is the measured int8 issue rate.
    pkm = mma_peaks(torch)
    out["tensor_peaks_mma_probe"] = pkm
    for m in (2048, 16384):
        tot_ops, tot_ms, tot_q, per_shape = 0.0, 0.0, 0.0, {}
        for (k, n) in [(2048, 2048), (2048, 8192), (8192, 2048)]:
            x = torch.randn(m, k, device="cuda", generator=g)
            x[:, torch.randperm(k, device="cuda", generator=g)[:max(1, k // 100)]] *= 20.0
            x = x.to(torch.bfloat16)
            w8 = torch.randint(-128, 128, (n, k), device="cuda", generator=g, dtype=torch.int8)
            cs = torch.rand(n, device="cuda", generator=g)
            bias = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
            x8, rs = ops.act_quant_per_token(x)
            ms = tm(lambda: ops.gemm_a8w8(x8, w8, rs, cs, 1.0, bias), reps=10, warm=3, graph=True)
            tot_q += tm(lambda: ops.act_quant_per_token(x), reps=10, warm=3, graph=True)
            tot_ops += 2.0 * m * n * k; tot_ms += ms
            per_shape[f"{k}x{n}"] = round(2.0 * m * n * k / ms / 1e9, 1)
        tops = tot_ops / tot_ms / 1e9
        out[f"a8w8_opt_m{m}"] = {"TOP/s": round(tops, 1), "ms": round(tot_ms, 3), "frac_int8_measured": round(tops / pkm["int8_tops_measured"], 3),
                                 "act_quant_ms": round(tot_q, 3), "TOP/s_with_act_quant": round(tot_ops / (tot_ms + tot_q) / 1e9, 1),
                                 "TOP/s_per_shape_KxN": per_shape}


def _wgrad_part(torch, ops, pk, out, tm, g):
    """Weight gradient dW += dY^T·X of the fine-tune step (OPT-1.3B at 2048 tokens, Llama-2-7B at 4096): this package's
    tcgen05 kernel against the library GEMM with beta = 1 that the trainer uses by default."""
    rows = {}
    for (m, n, k) in [(2048, 2048, 2048), (2048, 8192, 2048), (2048, 2048, 8192), (4096, 4096, 4096), (4096, 11008, 4096), (4096, 4096, 11008)]:
        dy = torch.randn(m, n, device="cuda", generator=g).to(torch.bfloat16)
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        dw = torch.zeros(n, k, device="cuda", dtype=torch.bfloat16)
        t_own = tm(lambda: ops.gemm_wgrad(dy, x, dw, accumulate=True), reps=10, warm=2)
        t_lib = tm(lambda: dw.addmm_(dy.t(), x), reps=10, warm=2)
        fl = 2.0 * m * n * k
        rows[f"M{m}_N{n}_K{k}"] = {"tcgen05_TFLOP/s": round(fl / t_own / 1e9, 1), "library_TFLOP/s": round(fl / t_lib / 1e9, 1),
                                   "frac_burst": round(fl / t_own / 1e9 / pk["bf16"], 3)}
        del dy, x, dw
    out["wgrad"] = rows


DECODE_M_LIST = (1, 8, 16, 64, 128, 512, 4096)


def _decode_part(torch, ops, pk, out, tm):
    # A16W4 forward at decode / small M over the four Llama shapes: bandwidth view (packed weights + qparams + activations).
    # One pass over the four layers is captured in a CUDA graph and replayed, as a decode loop would do: at these
    # sizes a launch from Python costs more than the kernel runs.
    layers = build_layers(torch, ops)
    for m in DECODE_M_LIST:
        xs = [L["x"][:m].contiguous() for L in layers]
        ys = [torch.empty(m, L["N"], device="cuda", dtype=torch.bfloat16) for L in layers]

        def one_pass():
            for L, x, y in zip(layers, xs, ys):
                ops.gemm_a16w4_fwd(x, L["codes"], L["s"], L["z"], None, L["N"], L["K"], out=y)

        one_pass(); torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_pass()
        ms_tot = tm(graph.replay, reps=20, warm=3)
        bytes_tot = sum(L["N"] * L["K"] / 2 + 4.0 * L["N"] * L["K"] / GROUP + 2.0 * m * (L["K"] + L["N"]) for L in layers)
        fl = sum(2.0 * m * L["N"] * L["K"] for L in layers)
        roof_ms = max(fl / (pk["bf16"] * 1e9), bytes_tot / (pk["hbm_gbs"] * 1e6))
        out[f"a16w4_fwd_m{m}"] = {"TFLOP/s": round(fl / ms_tot / 1e9, 2), "GB/s": round(bytes_tot / ms_tot / 1e6, 1),
                                  "frac_hbm": round(bytes_tot / ms_tot / 1e6 / pk["hbm_gbs"], 3), "ms": round(ms_tot, 4),
                                  "frac_roofline": round(roof_ms / ms_tot, 3),
                                  "timing": "CUDA graph replay of the 4 layers"}
        if m >= 16:                                       # grad-input dx = dy·deq(W) over the same layers
            dys = [L["dy"][:m].contiguous() for L in layers]
            dxs = [torch.empty(m, L["K"], device="cuda", dtype=torch.bfloat16) for L in layers]

            def one_pass_dgrad():
                for L, dy, dx in zip(layers, dys, dxs):
                    ops.gemm_a16w4_dgrad(dy, L["codes"], L["s"], L["z"], L["N"], L["K"], out=dx)

            one_pass_dgrad(); torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                one_pass_dgrad()
            ms_d = tm(graph.replay, reps=20, warm=3)
            out[f"a16w4_dgrad_m{m}"] = {"TFLOP/s": round(fl / ms_d / 1e9, 2), "ms": round(ms_d, 4),
                                        "frac_roofline": round(roof_ms / ms_d, 3), "timing": "CUDA graph replay of the 4 layers"}


def finetune_measurement(torch, arch="opt-1.3b", steps=10, warmup=2, micro_batch=4, seq=512, grad_accum=8, cuda_graph=True,
                         decode_batches=()):
    """Latent fine-tune step (the fine-tune configuration of the benchmark set): A16W4 int4 group-128 latent weights, seq 512, micro-batch 4,
    grad-accum 8 per rank, uniform random token ids, data-parallel over the ranks of this launch: the bf16
    gradient arena is all-reduced once per optimizer step, under the last backward pass and the optimizer step.  tokens/s = world * micro_batch * seq * grad_accum / step time.
    Token ids come from pinned host memory every step and the loss is read back (end-to-end through the module API)."""
    import torch.distributed as dist
    from latentq_llm_b200 import finetune as ft
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    model = ft.build_model(arch, "cuda", seed=1234)
    ft.quantize_decoder(model, lbit=4, gbit=16)
    opt, groups = ft.build_optimizer(model, lr=1e-4)
    tuner = ft.LatentFineTuner(model, opt, groups, grad_accum=grad_accum, cuda_graph=cuda_graph)
    vocab = ft.ARCHS[arch]["vocab_size"]
    host = [torch.randint(0, vocab, (micro_batch, seq), generator=torch.Generator().manual_seed(100 + rank * 1000 + i)).pin_memory()
            for i in range(grad_accum)]

    def one_step():
        batches = [h.to("cuda", non_blocking=True) for h in host]
        return float(tuner.step(batches))          # float(): device -> host read of the loss

    losses = [one_step() for _ in range(warmup)]
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        losses.append(one_step())
    e1.record(); torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda", dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    tokens = world * micro_batch * seq * grad_accum
    same = True
    if world > 1:
        from latentq_llm_b200.dp import replicas_identical
        qp = groups[0]["params"]                       # every quantized weight: packed codes and residual words
        same = replicas_identical([p.data for p in qp] + [p.residual.residual_int for p in qp
                                                           if hasattr(getattr(p, "residual", None), "residual_int")])
    # data-parallel efficiency measured in this run: the same step with the gradient exchange switched off (every rank
    # steps on its own gradients; done last, the replicas diverge from here on) against the step with it
    dp_eff, ms_local = None, None
    if world > 1:
        tuner.exchange = False
        one_step()
        dist.barrier(); torch.cuda.synchronize()
        e0.record()
        for _ in range(max(2, steps // 2)):
            one_step()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / max(2, steps // 2)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_local = float(t)
        dp_eff = round(ms_local / ms, 4)
    res = {"arch": arch, "tokens_per_s": round(tokens / ms * 1e3, 1), "ms_per_step": round(ms, 1), "world": world,
           "steps_timed": steps, "warmup_steps": warmup, "dp_efficiency": dp_eff,
           "ms_per_step_without_exchange": None if ms_local is None else round(ms_local, 1),
           "micro_batch": micro_batch, "seq": seq, "grad_accum": grad_accum, "loss_first": round(losses[0], 4),
           "loss_last": round(losses[-1], 4), "replica_codes_identical": same,
           "grad_arena_bytes": tuner.arena.flat.numel() * 2, "h2d_bytes_per_step": grad_accum * micro_batch * seq * 8,
           "micro_batch_fwd_bwd": "one captured CUDA graph, replayed" if cuda_graph else "eager"}
    if decode_batches:
        # greedy decode through the same quantized model (eval path of the module API, HF generate with a KV cache):
        # 512-token random prompts; tokens/s over the decode steps only (prefill timed separately and subtracted)
        model.eval()
        dec = {}
        from torch.nn.attention import SDPBackend, sdpa_kernel
        # (the cuDNN attention backend rebuilds its plan for every new KV length: ~5 ms of host time per layer and token)
        with torch.no_grad(), sdpa_kernel([SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]):
            for b in decode_batches:
                prompt = torch.randint(0, vocab, (b, 512), device="cuda")
                kw = dict(do_sample=False, use_cache=True, pad_token_id=0)
                model.generate(prompt, max_new_tokens=2, min_new_tokens=2, **kw)           # warm-up
                torch.cuda.synchronize(); t0 = time.perf_counter()
                model.generate(prompt, max_new_tokens=1, min_new_tokens=1, **kw)
                torch.cuda.synchronize(); t1 = time.perf_counter()
                model.generate(prompt, max_new_tokens=33, min_new_tokens=33, **kw)
                torch.cuda.synchronize(); t2 = time.perf_counter()
                dec[f"batch{b}"] = {"prefill_ms": round((t1 - t0) * 1e3, 1),
                                    "hf_generate_tokens_per_s": round(b * 32 / max(1e-9, (t2 - t1) - (t1 - t0)), 1)}
                # the same decode with the per-token step captured as one CUDA graph on a static KV cache
                from latentq_llm_b200.generate import GraphedGreedyDecoder
                gd = GraphedGreedyDecoder(model, batch=b, max_len=512 + 72)
                gd.generate(prompt, 4)                                                      # capture + warm-up
                torch.cuda.synchronize(); t0 = time.perf_counter()
                gd.generate(prompt, 1)
                torch.cuda.synchronize(); t1 = time.perf_counter()
                gd.generate(prompt, 65)
                torch.cuda.synchronize(); t2 = time.perf_counter()
                dec[f"batch{b}"]["graphed_tokens_per_s"] = round(b * 64 / max(1e-9, (t2 - t1) - (t1 - t0)), 1)
                del gd
                # the decode step as a chain of the library's own kernels (fused q|k|v and gate|up projections, RMSNorm,
                # RoPE + KV-cache write, single-query attention, silu*up), one CUDA graph; timed over graph replays only
                if ft.ARCHS[arch]["kind"] == "llama":
                    from latentq_llm_b200.generate import FusedLlamaGreedyDecoder
                    fd = FusedLlamaGreedyDecoder(model, batch=b, max_len=512 + 72)
                    fd.generate(prompt, 4)
                    torch.cuda.synchronize()
                    fd.generate(prompt, 2)
                    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    ev0.record()
                    for _ in range(64):
                        fd.graph.replay()
                    ev1.record(); torch.cuda.synchronize()
                    ms_tok = ev0.elapsed_time(ev1) / 64
                    dec[f"batch{b}"]["fused_tokens_per_s"] = round(b / ms_tok * 1e3, 1)
                    dec[f"batch{b}"]["fused_ms_per_step"] = round(ms_tok, 3)
                    del fd
                torch.cuda.empty_cache()
        res["greedy_decode"] = dec
        res["greedy_decode_note"] = ("512-token random prompts; hf_generate = the reference's route (eager loop, host-bound); "
                                     "graphed = decode step of the eager modules captured as one CUDA graph on a static KV cache; "
                                     "fused = decode step as nine library kernels per layer, one CUDA graph")
    del tuner, opt, model
    torch.cuda.empty_cache()
    return res


_CPU_DATA: dict = {}


def cpu_baseline(sample_m=512, reps=1):
    """The reference's CPU path for this workload (DeQfunc_4bit_g then input.mm(W.t()) / grad.mm(W), fp32,
    utils/quant.py:116-121,136-140) restated with the oracle, on a bounded sample: all four shapes at M=sample_m
    (the benchmark's M is 4096; the CPU path's rate does not depend on M beyond the weight dequantize)."""
    import numpy as np
    import torch
    import oracle as orc
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    data = _CPU_DATA.get(sample_m)
    if data is None:                                        # synthetic inputs, made once per process
        rng = np.random.default_rng(0)
        data = _CPU_DATA[sample_m] = []
        for (k, n) in LLAMA_SHAPES:
            data.append((k, n, rng.integers(-128, 128, n * k // 2, dtype=np.int8), np.full(n * k // GROUP, 0.008, np.float32),
                         np.full(n * k // GROUP, 8.0, np.float32),
                         torch.from_numpy(rng.standard_normal((sample_m, k)).astype(np.float32)),
                         torch.from_numpy(rng.standard_normal((sample_m, n)).astype(np.float32))))
    def deq(codes, s, z, n, k):
        """python_decompress + DeQfunc_4bit_g (utils/quant.py:12-19, 66-72) as the reference runs them on CPU tensors."""
        c = torch.from_numpy(codes)
        q = torch.stack([(c >> 4) % 16, c % 16], dim=1).reshape(-1, GROUP).to(torch.float32)
        return ((q - torch.from_numpy(z).view(-1, 1)) * torch.from_numpy(s).view(-1, 1)).view(n, k)

    k0, n0, c0, s0, z0 = data[0][:5]                       # the torch restatement against the oracle's, once
    assert np.array_equal(deq(c0[:4096], s0[:64], z0[:64], 2, 4096).numpy().ravel(), orc.a16w4_dequant(c0[:4096], s0[:64], z0[:64], GROUP))
    best, chk = float("inf"), 0.0
    for _ in range(reps):
        t0 = time.perf_counter()
        for (k, n, codes, s, z, x, dy) in data:
            y = x.mm(deq(codes, s, z, n, k).t())
            dx = dy.mm(deq(codes, s, z, n, k))             # backward dequantizes again (:136)
            chk += float(y[0, 0] + dx[0, 0])
        best = min(best, time.perf_counter() - t0)
    fl = step_flops(sample_m)
    return {"value": round(fl / best / 1e12, 4), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"all four (K,N) shapes at M={sample_m} (the benchmark's M is {M_TOKENS}), fwd+grad-input incl. weight "
                      f"dequantize, best of {reps}",
            "seconds": round(best, 3)}, chk


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    t_all = time.perf_counter()
    vals = []
    for _ in range(args.warmup):
        cpu_baseline(reps=1)
    for _ in range(args.steps):                             # every step is one bounded sample of the workload
        b, _ = cpu_baseline(reps=1)
        vals.append(b)
    secs = sum(v["seconds"] for v in vals)
    fl = step_flops(512) * len(vals)
    value = fl / secs / 1e12
    cb = dict(vals[-1]); cb["value"] = round(value, 4)
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(1e3 * secs / len(vals), 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": cb["sample"]},
            "cpu_baseline": cb, "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": round(time.perf_counter() - t_all, 1)}
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from latentq_llm_b200 import _lib, ops     # raises if the CUDA library is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    pk = peaks()

    layers = build_layers(torch, ops)
    for _ in range(max(args.warmup, 3)):
        run_step(ops, layers)
    torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    ms, launches = timed(torch, lambda: run_step(ops, layers), args.steps, barrier)
    clocks = sampler.stop() if sampler else None
    assert _lib.lib.lq_gemm_device_status(1) == 0, "a bounded device-side wait expired"

    # end-to-end: same GEMMs through the public call with HOST buffers (pinned), copies inside the timed region
    host = []
    for L in layers:
        host.append(dict(x=L["x"].cpu().pin_memory(), dy=L["dy"].cpu().pin_memory(),
                         y=torch.empty(M_TOKENS, L["N"], dtype=torch.bfloat16).pin_memory(),
                         dx=torch.empty(M_TOKENS, L["K"], dtype=torch.bfloat16).pin_memory()))
    h2d = sum(h["x"].numel() + h["dy"].numel() for h in host) * 2
    d2h = sum(h["y"].numel() + h["dx"].numel() for h in host) * 2

    # three streams: uploads, GEMMs (the current stream), downloads — PCIe is full duplex, so the input copy of one launch,
    # the GEMM of another and the result copy of a third run at the same time.  Every step still uploads every input and
    # downloads every result; a step ends when its last result is in host memory.
    cur, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
    consumed = [[torch.cuda.Event(), torch.cuda.Event()] for _ in layers]    # GEMM i has read its device input buffer

    def e2e_step():
        for i, (L, h) in enumerate(zip(layers, host)):
            for j, (dev_in, host_in, dev_out, host_out) in enumerate(((L["x"], h["x"], L["y"], h["y"]),
                                                                      (L["dy"], h["dy"], L["dx"], h["dx"]))):
                up = torch.cuda.Event()
                with torch.cuda.stream(s_in):
                    s_in.wait_event(consumed[i][j])              # the previous step's GEMM on this buffer
                    dev_in.copy_(host_in, non_blocking=True)
                    up.record()
                cur.wait_event(up)
                if j == 0:
                    ops.gemm_a16w4_fwd(dev_in, L["codes"], L["s"], L["z"], None, L["N"], L["K"], out=dev_out)
                else:
                    ops.gemm_a16w4_dgrad(dev_in, L["codes"], L["s"], L["z"], L["N"], L["K"], out=dev_out)
                consumed[i][j].record()
                s_out.wait_stream(cur)
                with torch.cuda.stream(s_out):
                    host_out.copy_(dev_out, non_blocking=True)
        cur.wait_stream(s_out)                                   # results of this step are on the host before the next GEMM overwrites them
        return launches_per_layer() * len(layers)

    e2e_step(); torch.cuda.synchronize()
    e2e_steps = max(2, min(args.steps, 10))
    ms_e2e, _ = timed(torch, e2e_step, e2e_steps, barrier)
    assert torch.equal(host[len(layers) // 2]["y"], layers[len(layers) // 2]["y"].cpu()) and torch.equal(host[-1]["dx"], layers[-1]["dx"].cpu()), \
        "end-to-end results in host memory differ from the device results"

    t = torch.tensor([ms, ms_e2e], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        fl = step_flops()
        value = world * fl * args.steps / ms / 1e9          # TFLOP/s, whole job
        e2e_value = world * fl * e2e_steps / ms_e2e / 1e9
        per_gpu = value / world
        line = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": WORKLOAD, "parallelism": "replicas only" if world > 1 else "single GPU",
                           "l2": "per-step working set ~1.1 GB of distinct buffers, larger than the 126 MB L2"},
                "roofline": roofline_entry(per_gpu, pk, clocks),
                "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": round(ms_e2e / e2e_steps, 3),
                        "pipeline": "pinned host buffers; upload, GEMM and download on three streams"},
                "gpu_launches": launches, "clocks": clocks}
        if world == 1 and not args.no_extra:
            line["extra"] = extra_measurements(torch, ops, pk)
            import oracle
            oracle.build()
            line["cpu_baseline"], _ = cpu_baseline()
    # the data-parallel fine-tune step runs on every rank (it has the path's one real exchange step)
    ft_res = None
    if not args.no_extra:
        del layers, host
        torch.cuda.empty_cache()
        try:
            ft_res = finetune_measurement(torch)
        except Exception as e:                      # the headline line must still be printed
            ft_res = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()
        try:                                        # Llama-2-7B architecture, seq 1024, micro-batch 4, one micro-batch per step
            ft7 = finetune_measurement(torch, arch="llama-2-7b", steps=10, warmup=2, micro_batch=4, seq=1024, grad_accum=1,
                                       decode_batches=(1, 16, 64) if rank == 0 else ())
        except Exception as e:
            ft7 = {"error": repr(e)[:300]}
    if rank == 0:
        if ft_res is not None:
            line.setdefault("extra", {})["finetune_opt1.3b"] = ft_res
            line["extra"]["finetune_llama2_7b"] = ft7
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary measurements and the CPU baseline")
    ap.add_argument("--only", default="", choices=["", "requant", "sweep", "stream", "a8w8", "decode", "decode_step", "wgrad", "mma_probe"],
                    help="run one family of the secondary measurements only (profiling a single kernel)")
    ap.add_argument("--numel", type=int, default=1 << 30, help="weights in the requantize measurement")
    ap.add_argument("--layers", type=int, default=4, help="--only decode_step: decoder layers of the 7B architecture to build")
    ap.add_argument("--batch", type=int, default=1, help="--only decode_step: sequences decoded together")
    ap.add_argument("--m", default="", help="--only decode: comma-separated token counts instead of the whole sweep")
    ap.add_argument("--shapes", default="", help="comma-separated indices into the shape list (profiling a smaller case)")
    args = ap.parse_args()
    if args.shapes:
        global LLAMA_SHAPES, WORKLOAD
        LLAMA_SHAPES = [LLAMA_SHAPES[int(i)] for i in args.shapes.split(",")]
        WORKLOAD += f" [subset {LLAMA_SHAPES}]"
    DECODE_STEP_ARGS.update(layers=args.layers, batch=args.batch)
    if args.m:
        global DECODE_M_LIST
        DECODE_M_LIST = tuple(int(v) for v in args.m.split(","))
    if args.only:
        import torch
        from latentq_llm_b200 import ops
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        print(json.dumps({"only": args.only, "extra": extra_measurements(torch, ops, peaks(), args.only, args.numel)}), flush=True)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
