/*
 * liblatentq — C ABI of the B200 (sm_100a) quantized-weight hot path.
 *
 * Every entry point takes raw DEVICE pointers plus explicit sizes, launches on
 * the given CUDA stream (cudaStream_t passed as void*, NULL = default stream),
 * returns 0 (LQ_OK) or a negative LQ_E* code, never throws, never aborts, and
 * never retains a pointer.  Nothing is allocated by the library: kernels that
 * need scratch memory take a caller-provided workspace (size from
 * lq_gemm_workspace_bytes).  Calls are asynchronous; the caller synchronises.
 *
 * Each declaration names the interface of FWkey/latentQ_LLM it replaces
 * (path:line inside that project).
 */
#ifndef LATENTQ_H
#define LATENTQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LQ_API __attribute__((visibility("default")))
#else
#define LQ_API
#endif

typedef void* lq_stream_t; /* cudaStream_t */

enum { LQ_OK = 0, LQ_EINVAL = -1, LQ_EUNSUPPORTED = -2, LQ_ECUDA = -3, LQ_ETIMEOUT = -4, LQ_EWORKSPACE = -5 };
enum { LQ_F32 = 0, LQ_BF16 = 1 };
enum { LQ_CODEC_NONE = 0, LQ_CODEC_UNIFORM16 = 1, LQ_CODEC_THREEFOLD = 2 };
enum { LQ_DITHER_HASH = 0, LQ_DITHER_EXPLICIT = 1, LQ_DITHER_PHILOX = 2 };

LQ_API int lq_version(void);
LQ_API const char* lq_status_string(int status);
/* cudaGetLastError-style text of the most recent LQ_ECUDA on this thread. */
LQ_API const char* lq_last_cuda_error(void);

/* ------------------------------------------------------------------------
 * Residual codecs: the five functions of the pybind module `MyQuantDequant`
 * (utils/cuda_src/multi_random_quant.cpp:38-54; kernels
 * utils/cuda_src/multi_random_quant_kernel.cu:9-334).  `x` holds
 * 8*n_words elements of dtype LQ_F32 / LQ_BF16; one int32 word packs 8
 * nibbles, element k at bits 28-4k.  The quantizers overwrite `x` with the
 * 0/1 carry flags like the reference does.
 * ------------------------------------------------------------------------ */
/* `quant`   (multi_random_quant.cpp:13-16, kernel .cu:9-128, launcher :345-361) */
LQ_API int lq_res3_quant(void* x, int dtype, int32_t* words, int64_t n_words,
                         int k1, float b1, int k2, float b2, int k3, float v0, lq_stream_t stream);
/* `dequant` (multi_random_quant.cpp:18-21, kernel .cu:130-217, launcher :384-399) */
LQ_API int lq_res3_dequant(const int32_t* words, void* x, int dtype, int64_t n_words,
                           int k1, float b1, int k2, float b2, int k3, lq_stream_t stream);
/* `uniform_quant`   (multi_random_quant.cpp:23-26, kernel .cu:241-294) */
LQ_API int lq_resu_quant(void* x, int dtype, int32_t* words, int64_t n_words, float v0, lq_stream_t stream);
/* `uniform_quant_s` (multi_random_quant.cpp:33-36, kernel .cu:219-239) */
LQ_API int lq_resu_quant_s(void* x, int dtype, int32_t* words, int64_t n_words, lq_stream_t stream);
/* `uniform_dequant` (multi_random_quant.cpp:28-31, kernel .cu:297-334) */
LQ_API int lq_resu_dequant(const int32_t* words, void* x, int dtype, int64_t n_words, lq_stream_t stream);
/* python_quant_linear / python_dequant_linear (utils/quant.py:765-788): the reference's only
 * CPU-runnable stochastic codec; `noise` is the U(-0.5,0.5) draw (fp32, n elements). */
LQ_API int lq_uniform16_encode(const float* r, const float* noise, int64_t n, int32_t* words, float* carry,
                               lq_stream_t stream);
LQ_API int lq_uniform16_decode(const int32_t* words, int64_t n_words, float* out, lq_stream_t stream);

/* ------------------------------------------------------------------------
 * Packing: python_compress / python_decompress (utils/quant.py:4-19; twins in
 * PTQ/quant/quant_linear.py:400-416).  byte i = (code[2i] << 4) + code[2i+1].
 * ------------------------------------------------------------------------ */
LQ_API int lq_pack_nibbles(const uint8_t* codes, int8_t* packed, int64_t n_codes, lq_stream_t stream);
LQ_API int lq_unpack_nibbles(const int8_t* packed, int8_t* codes, int64_t n_bytes, lq_stream_t stream);

/* Conversion between the two packed int4 layouts of the reference: nibble-pair int8 [N*K/2]
 * (QuantLinearA16W4.pack, PTQ/quant/quant_linear.py:455-470; the layout main0.py loads) and GPTQ int32 [K/8, N]
 * (QuantLinearGPTQ.pack, PTQ/quant/quant_linear.py:343-377).  Codes only; scales / zero points are small
 * [groups, N] <-> [N*groups] transposes done by the host code. */
LQ_API int lq_nibblepair_to_gptq(const int8_t* qweight_np, int32_t* qweight_gptq, int64_t N, int64_t K, lq_stream_t stream);
LQ_API int lq_gptq_to_nibblepair(const int32_t* qweight_gptq, int8_t* qweight_np, int64_t N, int64_t K, lq_stream_t stream);

/* DeQfunc_4bit_g (utils/quant.py:66-72).  qparams of dtype qp_dtype, one per `group` elements.
 * qp_dtype == LQ_BF16 reproduces the bf16 arithmetic of the GPU reference. */
LQ_API int lq_a16w4_dequant(const int8_t* qweight, const void* scales, const void* zeros, int qp_dtype,
                            void* out, int out_dtype, int64_t numel, int group, lq_stream_t stream);

/* Quantizer.find_params on x.view(-1, group) (PTQ/quant/quantizer.py:34-74; called per group at
 * PTQ/gptq.py:114-118): fp32 scale/zero per group; warp-shuffle min/max. */
LQ_API int lq_find_qparams(const void* x, int dtype, int64_t numel, int group, int maxq, int sym,
                           float* scales, float* zeros, lq_stream_t stream);

/* ------------------------------------------------------------------------
 * Latent-weight requantize.
 * ------------------------------------------------------------------------ */
typedef struct lq_requant_opts {
    int32_t codec;          /* LQ_CODEC_*: how the 4-bit residual is coded                      */
    int32_t dither;         /* LQ_DITHER_*: hash (CUDA reference), explicit buffer, or Philox    */
    int32_t math_dtype;     /* LQ_F32 / LQ_BF16: dtype the reference chain would run in          */
    int32_t res_round_bf16; /* cast the residual to bf16 before coding (utils/quant.py:726,737)  */
    int32_t has_residual;   /* 0 while ResidualTensor.init is True (utils/quant.py:833-836)      */
    int32_t mu_enc, mu_dec; /* three_fold_curve_4bit level used to encode / decode (:708-716)    */
    float v0;               /* hash-dither offset (the reference always passes 0, .cu:351)       */
    uint64_t seed;          /* Philox key                                                        */
    uint64_t stream_id;     /* Philox counter high words: (optimizer step, parameter id)         */
    const float* dither_buf;/* LQ_DITHER_EXPLICIT: one fp32 value in [-0.5,0.5] per element      */
} lq_requant_opts;

/* Qfunc_4bit_g_res (utils/quant.py:45-63): latent `w` -> packed codes + residual words. */
LQ_API int lq_a16w4_requant(const void* w, int w_dtype, const void* scales, const void* zeros, int qp_dtype,
                            int64_t numel, int group, const lq_requant_opts* opts,
                            int8_t* codes_out, int32_t* words_out, lq_stream_t stream);
/* One fused pass of MyAdam.update_step's weight path (utils/quant.py:1069-1073, 831-837, 1143):
 * latent = residual.add(DeQfunc_4bit_g(codes)) + delta ; codes, residual = Qfunc_4bit_g_res(latent).
 * In place on `codes` and `words`. */
LQ_API int lq_a16w4_fold_delta(int8_t* codes, int32_t* words, const void* delta, int delta_dtype,
                               const void* scales, const void* zeros, int qp_dtype,
                               int64_t numel, int group, const lq_requant_opts* opts, lq_stream_t stream);
/* Qfunc_8bit_res (utils/quant.py:88-103): per-row scale, codes int8 [rows, cols]. */
LQ_API int lq_a8w8_requant(const void* w, int w_dtype, const void* qscales, int qp_dtype,
                           int64_t rows, int64_t cols, const lq_requant_opts* opts,
                           int8_t* codes_out, int32_t* words_out, lq_stream_t stream);
LQ_API int lq_a8w8_fold_delta(int8_t* codes, int32_t* words, const void* delta, int delta_dtype,
                              const void* qscales, int qp_dtype, int64_t rows, int64_t cols,
                              const lq_requant_opts* opts, lq_stream_t stream);
/* Diagnostic (no counterpart in the reference): number of residual words the bf16 fast path of
 * lq_a16w4_fold_delta / lq_a16w4_requant handed to the generic code since the last reset (weights far outside
 * the quantization range, non-finite values).  Synchronises with the device. */
LQ_API int lq_fold_fallback_words(int reset, unsigned long long* count);
/* The library's Philox dither stream, materialised (test / debugging aid). */
LQ_API int lq_philox_dither(uint64_t seed, uint64_t stream_id, int64_t first_word, int64_t n_words, float* out,
                            lq_stream_t stream);

/* ------------------------------------------------------------------------
 * 8-bit optimizer-state codec: Qfunc_8bit_opt / DeQfunc_8bit_opt (utils/quant.py:22-41)
 * with `block` contiguous elements per (scale, t_max) pair (2048 or 128, :1038-1045).
 * ------------------------------------------------------------------------ */
LQ_API int lq_opt8_quant(const float* x, int64_t n, int block, uint8_t* q, float* scale, float* tmax,
                         lq_stream_t stream);
LQ_API int lq_opt8_dequant(const uint8_t* q, int64_t n, int block, const float* scale, const float* tmax,
                           float* x, lq_stream_t stream);

/* ------------------------------------------------------------------------
 * Fused optimizer step: MyAdam.update_step (utils/quant.py:1052-1148) in one pass.
 * ------------------------------------------------------------------------ */
typedef struct lq_adam_hyper {
    float beta1, beta2;          /* as torch rounds the Python floats to the op's fp32 math type            */
    float one_minus_beta1, one_minus_beta2;
    float eps;
    float neg_step_size;         /* -(lr * sqrt(1 - beta2^t) / (1 - beta1^t)), rounded once from double      */
} lq_adam_hyper;

/* One quantized A16W4 weight, everything in place (utils/quant.py:1056-1073 latent reconstruction, :1075-1105
 * 8-bit state decode + Adam in the gradient's dtype, :1113-1131 state re-encode, :1143 requantize):
 *   latent = residual.add(DeQfunc_4bit_g(codes));  m, v = decode(state1), decode(state2)^2;  Adam;
 *   state1, state2 = Qfunc_8bit_opt(m), Qfunc_8bit_opt(sqrt(v)+eps);  codes, residual = Qfunc_4bit_g_res(latent).
 * `grad` is [numel] in `grad_dtype` (the chain runs in that dtype when the qparams have it too, as torch's type
 * promotion would); `opt_block` is 2048 or 128 elements per (scale, t_max) pair.  weight_decay must be 0 (the
 * only value the reference's parameter groups use, main0.py:445-472).  The residual-curve statistics update of
 * :1107-1111 is not part of this call. */
LQ_API int lq_adam_a16w4_step(int8_t* codes, int32_t* words, const void* grad, int grad_dtype,
                              const void* scales, const void* zeros, int qp_dtype, int64_t numel, int group,
                              uint8_t* state1, float* scale1, float* tmax1,
                              uint8_t* state2, float* scale2, float* tmax2, int opt_block,
                              const lq_adam_hyper* hyper, const lq_requant_opts* opts, lq_stream_t stream);

/* The statistic of the residual-curve refresh (utils/quant.py:1107-1111) for the step about to be taken: stat_out
 * (fp32 [numel / 128]) receives, per run of 128 elements, the fp32 sum of abs(exp_avg) / denom after the moment
 * update (each quotient rounded to the gradient's dtype like the tensor op).  Reads the gradient and both 8-bit
 * states, changes nothing; the reference's per-group mean is stat_out / 128 for group size 128.  Call it before the
 * step of a refresh iteration: the level it selects is the one that step encodes with. */
LQ_API int lq_adam_moment_stat(const void* grad, int grad_dtype, int64_t numel,
                               const uint8_t* state1, const float* scale1, const float* tmax1,
                               const uint8_t* state2, const float* scale2, const float* tmax2, int opt_block,
                               const lq_adam_hyper* hyper, float* stat_out, lq_stream_t stream);
/* One quantized A8W8 weight (the `wbit == 8` branches of MyAdam.update_step, utils/quant.py:1070-1071, 1139-1141):
 * latent = residual.add(codes * qscales[row]); Adam; states re-encoded; codes, residual = Qfunc_8bit_res(latent).
 * codes int8 [rows, cols], one scale per row, cols a multiple of 8. */
LQ_API int lq_adam_a8w8_step(int8_t* codes, int32_t* words, const void* grad, int grad_dtype,
                             const void* qscales, int qp_dtype, int64_t rows, int64_t cols,
                             uint8_t* state1, float* scale1, float* tmax1,
                             uint8_t* state2, float* scale2, float* tmax2, int opt_block,
                             const lq_adam_hyper* hyper, const lq_requant_opts* opts, lq_stream_t stream);

/* GradientQTensor (utils/quant.py:846-921): the optional 8-bit stochastic gradient accumulator.
 * first != 0 is set_value(): scale[row] = clamp(4 * absmax(row), 1e-5) / 127 (stored in `dtype`), then
 * qdata = clamp(round(fdata / scale + noise), -128, 127); first == 0 is add_(): fdata <- qdata * scale + fdata
 * first, scale unchanged.  noise comes from opts->dither (LQ_DITHER_EXPLICIT: opts->dither_buf, one fp32 value per
 * element; LQ_DITHER_PHILOX: opts->seed / opts->stream_id); no other field of opts is read.  cols a multiple of 8. */
LQ_API int lq_gradq_accumulate(const void* fdata, int dtype, int64_t rows, int64_t cols, int8_t* qdata, void* scale,
                               int first, const lq_requant_opts* opts, lq_stream_t stream);
/* get_value(): out = qdata.to(dtype) * scale[row]. */
LQ_API int lq_gradq_dequant(const int8_t* qdata, const void* scale, int dtype, int64_t rows, int64_t cols, void* out,
                            lq_stream_t stream);

/* Many small dense bf16 parameters with bf16 optimizer states (numel < 65536, utils/quant.py:1020-1027) in one
 * launch.  `table` is a DEVICE array of n_tensors records {param, grad, state1, state2, numel}; state2 holds
 * sqrt(v)+eps as in the reference (:1133-1135).  All four arrays of a record are bf16 and 16-byte aligned. */
typedef struct lq_dense_slot {
    void* param; const void* grad; void* state1; void* state2; int64_t numel;
} lq_dense_slot;
LQ_API int lq_adam_dense_multi(const lq_dense_slot* table, int n_tensors, int64_t max_numel,
                               const lq_adam_hyper* hyper, lq_stream_t stream);

/* ------------------------------------------------------------------------
 * Activation quantizers for the A8W8 path.
 * ------------------------------------------------------------------------ */
/* quantize_activation_per_token_absmax (PTQ/quant/quant_linear.py:520-528): bf16 x[M,K] ->
 * int8 + fp32 scale per token (computed in bf16 like the reference's in-place ops). */
LQ_API int lq_act_quant_per_token(const void* x, int64_t M, int64_t K, int8_t* x8, float* a_scale,
                                  lq_stream_t stream);
/* QLinearFunctionA8W8_dynamic.forward quantizer (utils/quant.py:260-266): clampv = max(x) computed
 * on device into clampv_out (fp32[1]); x8 = clamp(round(x*127/clampv)). */
LQ_API int lq_act_quant_per_tensor(const void* x, int64_t n, float* clampv_out, int8_t* x8, lq_stream_t stream);

/* ------------------------------------------------------------------------
 * GEMMs (tcgen05 / TMEM; TMA-staged operands).  Row-major everywhere.
 * ------------------------------------------------------------------------ */
enum { LQ_GEMM_A16W4_FWD = 0, LQ_GEMM_A16W4_DGRAD = 1, LQ_GEMM_A8W8 = 2 };
/* Bytes of caller-provided scratch the GEMM of that kind/shape may use (split-K partial sums; with LQ_GEMM_BALANCE=1
 * in the environment the partial sums of the shared-tile forward plan, which falls back to whole tiles when the
 * workspace given is smaller). */
LQ_API size_t lq_gemm_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K);

/* QLinearFunctionW4.forward (utils/quant.py:116-121): y[M,N] = x[M,K] · deq(qweight)[N,K]ᵀ (+ bias),
 * deq = DeQfunc_4bit_g with bf16 scales/zeros [N*K/group].  x, y, bias bf16. */
LQ_API int lq_gemm_a16w4_fwd(const void* x, const int8_t* qweight, const void* scales, const void* zeros,
                             const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group,
                             void* workspace, size_t workspace_bytes, lq_stream_t stream);
/* QLinearFunctionW4.backward grad_input (utils/quant.py:139-140): dx[M,K] = dy[M,N] · deq(qweight)[N,K]. */
LQ_API int lq_gemm_a16w4_dgrad(const void* dy, const int8_t* qweight, const void* scales, const void* zeros,
                               void* dx, int64_t M, int64_t N, int64_t K, int group,
                               void* workspace, size_t workspace_bytes, lq_stream_t stream);
/* torch_int._CUDA.linear_a8_w8_bbf16_obf16 (call sites utils/quant.py:181-389,
 * PTQ/quant/quant_linear.py:709-711): x8[M,K] · w8[N,K]ᵀ with int32 accumulation.
 *   y[m,n] = bf16( acc * row_scale[m] * col_scale[n] * alpha + bias[n] )
 * row_scale (fp32[M]) / col_scale (fp32[N]) / bias (bf16[N]) may be NULL (treated as 1 / 1 / 0);
 * alpha alone reproduces the torch_int call.  acc_out (int32[M,N]) may be NULL; when given the
 * raw accumulators are stored as well. */
LQ_API int lq_gemm_a8w8(const int8_t* x8, const int8_t* w8, const float* row_scale, const float* col_scale,
                        float alpha, const void* bias, void* y, int32_t* acc_out,
                        int64_t M, int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                        lq_stream_t stream);

/* Decode-sized forward (M <= 2, K = 4096, group 128) with the residual add and the RMSNorm in front of it folded into the
 * kernel's token staging (PTQ/quant/triton_norm.py:7-39 followed by the int4 matmul of PTQ/quant/fused_attn.py:164-204 /
 * fused_mlp.py:84-168): x = RMSNorm(h + delta) * gamma computed as lq_add_rmsnorm computes it (bit for bit), then
 * y[M,N] = x . deq(qweight)^T, or with silu_pair != 0 (qweight = gate | up, N = 2 I rows) y[M,I] = silu(gate) * up.
 * delta may be NULL (then h_out is not written); otherwise h_out receives h + delta and must be a buffer other than h
 * (every CTA reads h).  Returns LQ_EUNSUPPORTED for other shapes, and for launches with no more 16-row blocks than
 * persistent CTAs (two per SM), which another kernel serves: run lq_add_rmsnorm and the GEMM separately. */
LQ_API int lq_gemm_a16w4_fwd_rmsnorm(const void* h, const void* delta, const void* gamma, float eps, int hf_rounding, void* h_out,
                                     const int8_t* qweight, const void* scales, const void* zeros, void* y, int64_t M, int64_t N,
                                     int64_t K, int group, int silu_pair, lq_stream_t stream);

/* Decode-sized q|k|v projection (M <= 16) with the rotary embedding and the KV-cache write as its epilogue
 * (fused QuantLinear of PTQ/quant/fused_attn.py:164-204, triton_rotate_half_ fused_attn.py:8-58 and the cache append
 * fused_attn.py:124-140): one launch leaves what lq_gemm_a16w4_fwd followed by lq_rope_kv_store leaves, bit for bit -
 * qkv[M, (Hq + 2 Hkv) hd] with q rotated and k, v as projected, rotated k and v in the caches
 * [batch, kv head, max_len, hd] at positions[m] (batch = m / tokens_per_seq).  The kernel pairs weight row i of a head
 * with row i + hd/2 in one MMA block so that a thread holds both halves of a rotation.
 * Tokens: x[M,K] when gamma is NULL; otherwise RMSNorm(h + delta) * gamma computed in the token staging exactly as
 * lq_gemm_a16w4_fwd_rmsnorm does (same arguments, same shape limits).  LQ_EUNSUPPORTED for M > 16, hd not a multiple of
 * 16, or K / group the row-block decode kernels do not serve: run the GEMM and lq_rope_kv_store then. */
LQ_API int lq_gemm_a16w4_fwd_qkv_rope(const void* x, const void* h, const void* delta, const void* gamma, float eps,
                                      void* h_out, const int8_t* qweight, const void* scales, const void* zeros, void* qkv,
                                      const int64_t* positions, const float* inv_freq, void* k_cache, void* v_cache,
                                      int64_t M, int Hq, int Hkv, int hd, int64_t K, int group, int64_t max_len,
                                      int tokens_per_seq, int hf_rounding, lq_stream_t stream);

/* QLinearFunctionW4.backward grad_weight (utils/quant.py:141-142) and its accumulation over micro-batches by the
 * backward hook (:408-411): dw[N,K] (+)= dy[M,N]^T · x[M,K], all bf16 row-major, fp32 accumulation in tensor memory.
 * accumulate != 0: dw = bf16(fp32(dw) + product), one rounding, what a GEMM with beta = 1 computes; 0: dw = bf16(product).
 * Both operands are read by TMA as 64 x 64 boxes and fed to tcgen05.mma MN-major (no transpose pass).  N, K multiples of 8. */
LQ_API int lq_gemm_wgrad(const void* dy, const void* x, void* dw, int64_t M, int64_t N, int64_t K, int accumulate,
                         lq_stream_t stream);

/* Forward GEMM for callers that cannot allocate device memory (no counterpart in the reference).
 * Same arithmetic and arguments as lq_gemm_a16w4_fwd minus the workspace: split-K partial sums go into an
 * 8 MiB array built into the library (lq_gemm_a16w4_fwd_static_max_bytes), which every GPU that loads the
 * library keeps resident until exit.  It is meant for code that runs under a framework-owned memory pool,
 * for latency-critical loops that cannot afford the device-wide synchronisation an allocation implies, and
 * for plugin hosts that forbid allocations after start-up.  No cudaMalloc/cudaFree or allocating library
 * routine is called.  Shapes whose split-K plan needs more than the built-in array return LQ_EWORKSPACE
 * (lq_last_cuda_error() says why); use the workspace variant for those.  The first call on each device
 * looks up the array's device address (one runtime query, made with that device current): make that first
 * call before starting any stream capture.  All calls share the one array and it keeps whatever the last
 * call left in it; nothing in it needs clearing, but two calls that overlap on the GPU (different streams
 * without an ordering between them) race on it and must be serialised by the caller. */
LQ_API size_t lq_gemm_a16w4_fwd_static_max_bytes(void);
LQ_API int lq_gemm_a16w4_fwd_static(const void* x, const int8_t* qweight, const void* scales, const void* zeros,
                                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group,
                                    lq_stream_t stream);
/* Diagnostic for the entry point above (no counterpart in the reference): copies n_floats fp32 partial sums,
 * starting at element first_float, out of the built-in array of the CURRENT device into host memory.
 * Synchronises with the device; allocates nothing. */
LQ_API int lq_gemm_a16w4_fwd_static_peek(float* host_out, size_t first_float, size_t n_floats);

/* Every device-side wait in the GEMM kernels is bounded; when one expires the kernel gives up cleanly and
 * raises a device flag.  This call synchronises with the device, returns LQ_ETIMEOUT if the flag is set
 * (LQ_OK otherwise) and clears it when `reset` is non-zero.  (No counterpart in the reference.) */
LQ_API int lq_gemm_device_status(int reset);
/* Phase profile of the GEMM kernels (no counterpart in the reference).  Synchronises with the device, copies
 * the 16 cycle counters accumulated since the last call into out16 (may be NULL), clears them and switches
 * collection on/off.  Counters (summed over CTAs): [0] producer waiting for a free stage, [1] MMA issuer
 * waiting for TMA data, [2] MMA issuer waiting for the dequantised tile, [3] MMA issuer waiting for a free
 * accumulator, [4] MMA role total, [5] dequant waiting for TMA data, [6] dequant role total,
 * [7] epilogue waiting for an accumulator, [8] epilogue role total, [9] number of CTAs. */
LQ_API int lq_gemm_profile(int enable, unsigned long long* out16);

/* Decode chain switch (no counterpart in the reference).  While enabled, the decode-sized forward (M <= 16) and the
 * decode-side kernels below are launched with programmatic stream serialization: a kernel may start, and the forward
 * may fetch its WEIGHTS, while the previous kernel in the stream is still running; activations written by that kernel
 * are read only after it has completed.  Enable it only around chains whose weights are not written by the previous
 * kernel in the stream (a decode step).  Default: off.  Process-wide; returns the previous setting. */
LQ_API int lq_decode_chain(int enable);

/* ------------------------------------------------------------------------
 * Decode-side operations around the GEMMs of a Llama-architecture layer (bf16 everywhere).  hf_rounding != 0
 * rounds every intermediate to bf16 like the eager modules' tensor ops; 0 keeps fp32 up to the final cast like the
 * reference's Triton kernels.
 * ------------------------------------------------------------------------ */
/* Residual add + RMSNorm (PTQ/quant/triton_norm.py:7-39; LlamaRMSNorm): if delta != NULL, h[M,K] += delta first
 * (in place); y = h * rsqrt(mean(h^2) + eps) * gamma[K]. */
LQ_API int lq_add_rmsnorm(void* h, const void* delta, const void* gamma, float eps, void* y, int64_t M, int64_t K,
                          int hf_rounding, lq_stream_t stream);
/* Rotate-half RoPE on the q and k heads of a fused projection output (PTQ/quant/fused_attn.py:8-58, 124-129):
 * qkv[M, (Hq + 2*Hkv) * hd] = q | k | v per token; q is rotated in place, rotated k and v are written into the caches
 * [batch, Hkv, max_len, hd] at positions[m] (int64, one per token; batch index = m / tokens_per_seq).
 * inv_freq: hd/2 fp32 frequencies (theta^(-2i/hd)). */
LQ_API int lq_rope_kv_store(void* qkv, const int64_t* positions, const float* inv_freq, void* k_cache, void* v_cache,
                            int64_t M, int tokens_per_seq, int Hq, int Hkv, int hd, int64_t max_len, int hf_rounding,
                            lq_stream_t stream);
/* Single-query attention over the cache (the reference calls F.scaled_dot_product_attention,
 * PTQ/quant/fused_attn.py:148-149): out[b, h*hd..] = softmax(q[b,h]·K[b,hk,0..positions[b]] * scale) · V.
 * q: row b at q + b*q_row_stride elements, heads contiguous.  hd = 64 or 128.  The workspace holds the partial results
 * of the key-range splits and, behind them, one ticket counter per (batch, head); the counters must be ZERO before the
 * first call and are left zero by every call.  Their offset depends on B, Hq, hd and max_len: clear a workspace before
 * using it with another shape. */
LQ_API size_t lq_decode_attention_workspace_bytes(int64_t B, int Hq, int hd, int64_t max_len);
LQ_API int lq_decode_attention(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                               const int64_t* positions, void* out, int64_t B, int Hq, int Hkv, int hd, int64_t max_len,
                               float scale, void* workspace, size_t workspace_bytes, lq_stream_t stream);
/* Fused gate | up projection of a decode step (PTQ/quant/fused_mlp.py:84-168: C = silu(A·B1) * (A·B2) in one kernel):
 * qweight holds 2*I weight rows, gate rows first; act[M, I] = silu(x·Wgate^T) * (x·Wup^T), both products rounded to
 * bf16 first like the separate projections.  Decode-sized only (M <= 16, K a multiple of 256, group 128 or 256);
 * other shapes return LQ_EUNSUPPORTED: use lq_gemm_a16w4_fwd into [M, 2I] and lq_silu_mul. */
LQ_API int lq_gemm_a16w4_fwd_silu(const void* x, const int8_t* qweight, const void* scales, const void* zeros, void* act,
                                  int64_t M, int64_t I, int64_t K, int group, int hf_rounding, lq_stream_t stream);
/* End of a greedy decode step (the argmax + embedding look-up of HF generate's loop that the reference drives,
 * generate.py:150-190) in one launch: tok[b] = argmax over logits[b, 0..V) (bf16, row stride logits_stride elements; the
 * first maximum, NaN counted as the largest value, as torch.argmax); positions[b] += 1 when positions is not NULL;
 * h[b, 0..D) = embed[tok[b], 0..D) when embed is not NULL (D a multiple of 8, both 16-byte aligned). */
LQ_API int lq_argmax_embed(const void* logits, int64_t logits_stride, int64_t B, int64_t V, const void* embed, int64_t D,
                           int64_t* tok, int64_t* positions, void* h, lq_stream_t stream);
/* act[M, I] = silu(gate_up[M, 0:I]) * gate_up[M, I:2I] (epilogue of PTQ/quant/fused_mlp.py:84-168; LlamaMLP). */
LQ_API int lq_silu_mul(const void* gate_up, void* act, int64_t M, int64_t I, int hf_rounding, lq_stream_t stream);

/* Issue-rate microbenchmark of the tensor cores (no counterpart in the reference): `ctas` CTAs each issue n_mma
 * tcgen05.mma instructions of shape 128 x n x (32 bytes of k) — kind LQ_GEMM_A8W8: int8 operands, 32 k; otherwise
 * bf16, 16 k — on operands resident in shared memory (a_in_tmem != 0: bf16 A operand in tensor memory), rotating over
 * n_acc independent accumulators (n_acc * n <= 256).  The measured int8 / bf16 ceilings that the GEMM rooflines are
 * quoted against come from this call.  With max_cycles_out == NULL the launch is asynchronous (time it with events);
 * otherwise the call synchronises and returns the longest per-CTA cycle count of the run. */
LQ_API int lq_mma_issue_rate(int kind, int a_in_tmem, int n, int n_acc, int n_mma, int ctas,
                             unsigned long long* max_cycles_out, lq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LATENTQ_H */
