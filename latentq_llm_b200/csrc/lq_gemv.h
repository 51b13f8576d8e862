// Interface between the GEMM dispatcher and the decode-sized (M <= 16) forward kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lq {

struct SkinnyParams {
    const __nv_bfloat16* x;        // [M, K]
    const uint8_t* qweight;        // packed nibble pairs, K/2 bytes per row
    const __nv_bfloat16* scales;   // [N * K / group]
    const __nv_bfloat16* zeros;
    const __nv_bfloat16* bias;     // [N] or null
    __nv_bfloat16* out;            // [M, N]
    float* partial;                // [splits][M][N] when splits > 1
    int M, N, K, group, splits, chunks_per_split;
    // Paired rows (fused gate | up projection, row-block kernels only): pair_stride > 0 makes fragment rows 0..7 of a
    // block the weight rows f..f+7 and fragment rows 8..15 the rows pair_stride + f.., so that one thread holds
    // gate[f] and up[f] of a token; the output is act[M, N] = silu(gate) * up with N = pair_stride features.
    int pair_stride;
    int hf_rounding;               // pair epilogue: round silu(gate) to bf16 before the product (eager-module chain)
    // Fused residual add + RMSNorm in front (streaming kernel, K = 4096 only): when norm_gamma is set the tokens are not
    // read from x but computed by every CTA as RMSNorm(norm_h + norm_delta) * norm_gamma, exactly as lq_add_rmsnorm
    // computes them (same thread-to-element mapping, same order of the sum of squares); CTA 0 also writes the updated
    // residual norm_h + norm_delta to norm_h_out (a buffer other than norm_h: the other CTAs still read norm_h).
    const __nv_bfloat16* norm_h;
    const __nv_bfloat16* norm_delta;   // or null
    const __nv_bfloat16* norm_gamma;
    __nv_bfloat16* norm_h_out;         // or null when norm_delta is null
    float norm_eps;
    int norm_hf;
    // Fused rotary embedding + KV-cache write behind a q|k|v projection (row-block kernels): rope_hd > 0 pairs weight
    // row i of a head with row i + hd/2 of the same head in one MMA block (pair_stride = hd/2, N = pairs), so that one
    // thread holds both halves of a rotation.  out is the [M, (Hq + 2 Hkv) hd] projection buffer: q is written rotated,
    // k and v as projected; rotated k and v also go to the caches [batch, kv head, max_len, hd] at the token's
    // position.  Same arithmetic as lq_rope_kv_store on the bf16 projection.
    const long long* rope_pos;         // [M]
    const float* rope_inv_freq;        // [hd / 2]
    __nv_bfloat16* rope_k;
    __nv_bfloat16* rope_v;
    int rope_hd, rope_hq, rope_hkv, rope_max_len, rope_tps;
};

// split-K plan of the skinny kernel: returns 64-k chunks per split and writes the number of splits
int skinny_chunks_per_split(int64_t N, int64_t K, int* splits_out);
int launch_skinny_fwd(const SkinnyParams& p, cudaStream_t st);
// row-block variant: one launch, no workspace (splits / chunks_per_split / partial are ignored)
bool skinny_rows_supported(int64_t K, int group);
int launch_skinny_rows(const SkinnyParams& p, cudaStream_t st);
// true when launch_skinny_rows would take the streaming kernel with the fused-norm staging for this shape
bool skinny_norm_supported(int64_t M, int64_t K, int group);

}  // namespace lq
