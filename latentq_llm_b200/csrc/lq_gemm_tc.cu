// tcgen05 / TMEM GEMMs of liblatentq (sm_100a):
//   A16W4 forward      y[M,N]  = x[M,K]  · deq(Wq)[N,K]^T      (QLinearFunctionW4.forward,  utils/quant.py:116-121)
//   A16W4 grad-input   dx[M,K] = dy[M,N] · deq(Wq)[N,K]        (QLinearFunctionW4.backward, utils/quant.py:139-140)
//   A8W8               y[M,N]  = x8[M,K] · w8[N,K]^T, int32 accumulate, scaled epilogue
//                                                               (torch_int linear_a8_w8_bbf16_obf16 call sites, utils/quant.py:181-389)
//
// One persistent, warp-specialised kernel template.  The weight-derived operand is always the MMA "A"
// operand (128 rows per tile: output features for forward / int8, input features for grad-input), the
// token-side operand is "B" (16..256 tokens per tile), so the accumulator lives in TMEM as
// [128 lanes = weight rows] x [tokens] and one dequantised weight tile is reused by up to 256 tokens.
//
//   warp 0      : TMA producer   (token tile + raw packed int4 tile, or both int8 tiles)
//   warp 1      : MMA issuer     (one elected thread issues tcgen05.mma; owns TMEM alloc/dealloc)
//   warps 2..5  : epilogue       (tcgen05.ld -> scale/bias -> bf16 / partial sums -> global)
//   warps 6..21 : dequant        (A16W4 only: raw int4 in smem -> bf16((q-z)*s) -> 128B-swizzled MMA tile)
//
// Forward and grad-input share the dequant stage: a row of W[N,K] always becomes 128-byte rows of the
// swizzled tile; forward describes that tile to the tensor core as K-major, grad-input as MN-major.
//
// Every mbarrier wait is bounded (clock64 budget).  On expiry the CTA raises an abort flag in shared
// memory, all roles leave their loops, in-flight bulk copies are given time to land, TMEM is freed and a
// global status word is set (read back with lq_gemm_device_status).
#include <cuda.h>
#include <cstdlib>

#include "lq_common.cuh"
#include "lq_gemv.h"
#include "lq_tc.cuh"

namespace lq {

enum { KIND_FWD = LQ_GEMM_A16W4_FWD, KIND_DGRAD = LQ_GEMM_A16W4_DGRAD, KIND_I8 = LQ_GEMM_A8W8, KIND_WGRAD = 3 };

constexpr int ROW_BYTES = 128;        // one swizzle row
constexpr int A_TILE_BYTES = TILE_R * ROW_BYTES;
constexpr int RAW_BYTES = 4096;       // packed int4 bytes per stage (128 rows x 64 k, or 64 rows x 128 k)
constexpr int NUM_DQ_WARPS = 16;          // 512 dequant threads, 8 packed bytes (16 weights) each per stage
#ifndef LQ_MAX_STAGES
#define LQ_MAX_STAGES 8
#endif
constexpr int MAX_STAGES = LQ_MAX_STAGES;

__device__ int g_gemm_status;   // 0 = fine, 1 = a bounded wait expired in some CTA
// Optional phase profile (lq_gemm_profile): cycles summed over CTAs.
//  [0] producer waiting for a free stage   [1] MMA waiting for TMA data   [2] MMA waiting for the dequantised tile
//  [3] MMA waiting for a free accumulator  [4] MMA role total             [5] dequant waiting for TMA data
//  [6] dequant role total                  [7] epilogue waiting for an accumulator  [8] epilogue role total  [9] CTAs
//  balanced mode, lane quarter 0: [10] publishing partial sums (incl. ticket)  [11] adding a tile's parts up
//  (with its epilogue)  [12] tiles added up  [14] hand-over copies
__device__ unsigned long long g_gemm_prof[16];
__device__ int g_gemm_prof_on;

// ---------------------------------------------------------------------------------------------
// Kernel parameters
// ---------------------------------------------------------------------------------------------
struct GemmParams {
    int M;            // tokens
    int R;            // weight-side rows of the output (N for fwd / int8, K for dgrad)
    int C;            // contraction length (K for fwd / int8, N for dgrad)
    int wcols;        // in-features K of the weight matrix (row length of W)
    int group;        // A16W4 group size along K
    int r_tiles, t_tiles, splits, kb_total, kb_per_split;
    const __nv_bfloat16* scales;   // [N*K/group]
    const __nv_bfloat16* zeros;
    const __nv_bfloat16* bias;     // [R] or null
    const float* row_scale;        // int8: per token, or null
    const float* col_scale;        // int8: per output channel, or null
    float alpha;
    __nv_bfloat16* out;            // [M, R]
    int32_t* acc_out;              // int8: raw accumulators [M, R] or null
    void* partial;                 // split-K partial sums [splits][M][R] (fp32 / int32); balanced mode: slots + flags
    // balanced mode (SK), see SegWalk
    int sk_full;                   // tiles computed whole (a multiple of the grid size), the first ones
    int sk_rem;                    // shared tiles behind them, one owner CTA each (CTA j owns shared tile j)
    int sk_h;                      // k-blocks of a shared tile its owner computes (the head); the rest is its tail
    int sk_helpers;                // CTAs sk_rem .. sk_rem + sk_helpers - 1 share out the tails
    int sk_q, sk_r;                // tail units / helpers and tail units % helpers (helper h starts at unit h * q + h * r / helpers)
    int sk_pmax;                   // partial-sum slots per shared tile
    int accumulate;                // weight gradient: out += product (rounded once from the fp32 sum) instead of out = product
    const uint4* qpt;              // QPT kernels: per-column group parameters, packed for the dequant (see k_w4_qp_transpose)
};

// One CTA's share of the work as a sequence of segments (a tile and a range of its k-blocks).
//   tile-cyclic (SK = false): items blockIdx.x, blockIdx.x + gridDim.x, ...; an item is one (row tile, token tile,
//     split) and its whole k range.
//   balanced (SK = true): the first `sk_full` tiles are computed whole, tile-cyclic.  Each of the `sk_rem` tiles behind
//     them (fewer than the grid has CTAs) is shared: its owner, CTA j for shared tile j, computes the head
//     [0, sk_h) of its k range as its last piece of work, and the tails [sk_h, kb_total) of all shared tiles, laid end
//     to end as "tail units", are dealt in equal contiguous ranges to the helper CTAs, which have no tile of their own
//     left.  The host sizes the head so that the helpers are done a few k-blocks before the owners: an owner normally
//     finds its tile's other parts already published and adds them up in its epilogue.
struct Seg { int r_tile, t_tile, split, kb0, kb1; };
// Balanced mode: first tail unit of helper h, floor(units * h / helpers).
__device__ __forceinline__ int sk_helper_first(const GemmParams& p, int h) { return h * p.sk_q + (h * p.sk_r) / p.sk_helpers; }
// Balanced mode: the helper whose range holds tail unit u.
__device__ __forceinline__ int sk_helper_of(const GemmParams& p, int u) {
    int h = min(p.sk_helpers - 1, u / p.sk_q);
    while (sk_helper_first(p, h) > u) --h;
    return h;
}
template <bool SK>
struct SegWalk {
    int pos, end;       // tile-cyclic: next item, number of items; balanced: next whole tile, then this helper's tail units
    bool whole, owner;  // balanced: still in the whole tiles; an owned head is still to come
    __device__ __forceinline__ explicit SegWalk(const GemmParams& p) {
        pos = (int)blockIdx.x;
        if (SK) {
            end = p.sk_full; whole = true; owner = (int)blockIdx.x < p.sk_rem;
        } else {
            end = p.r_tiles * p.t_tiles * p.splits; whole = false; owner = false;
        }
    }
    __device__ __forceinline__ bool next(const GemmParams& p, Seg& s) {
        if (SK) {
            int tile;
            if (whole) {
                if (pos < end) {
                    tile = pos; pos += (int)gridDim.x; s.kb0 = 0; s.kb1 = p.kb_total;
                } else {
                    whole = false;
                    const int h = (int)blockIdx.x - p.sk_rem;
                    if (!owner && h < p.sk_helpers) { pos = sk_helper_first(p, h); end = sk_helper_first(p, h + 1); }
                    else { pos = end = 0; }
                }
            }
            if (!whole) {
                const int tail = p.kb_total - p.sk_h;
                if (owner) {
                    owner = false; tile = p.sk_full + (int)blockIdx.x; s.kb0 = 0; s.kb1 = p.sk_h;
                } else if (pos < end) {
                    const int j = pos / tail;
                    tile = p.sk_full + j; s.kb0 = p.sk_h + (pos - j * tail); s.kb1 = min(p.kb_total, s.kb0 + (end - pos));
                    pos += s.kb1 - s.kb0;
                } else {
                    return false;
                }
            }
            s.r_tile = tile % p.r_tiles; s.t_tile = tile / p.r_tiles; s.split = 0;
            return true;
        }
        if (pos >= end) return false;
        s.r_tile = pos % p.r_tiles; s.t_tile = (pos / p.r_tiles) % p.t_tiles; s.split = pos / (p.t_tiles * p.r_tiles);
        s.kb0 = s.split * p.kb_per_split; s.kb1 = min(p.kb_total, s.kb0 + p.kb_per_split);
        pos += (int)gridDim.x;
        return true;
    }
};

// RT = weight-row tiles (of 128 rows) a CTA computes against one token tile.  RT = 2 halves the token-tile
// bytes fetched from L2 per flop (the dominant operand traffic) at the cost of a shallower pipeline.
// TA = the dequantised weight tile is written to tensor memory (tcgen05.st) and read by the MMA from there instead
// of from shared memory: the 128 x 64 bf16 tile of a stage takes 32 TMEM columns, and per MMA the shared-memory
// pipe no longer carries its 4 KB write and 4 KB read (the kernel is shared-memory-bandwidth bound otherwise).
constexpr int TA_COLS_PER_STAGE = 32;
constexpr int FIX_COLS = 16;                                         // balanced mode: token columns per hand-over copy
constexpr int FIX_COPY_BYTES = FIX_COLS * 32 * 4;                    // one lane quarter of them as fp32: 2 KB
constexpr int FIX_RING = 8;                                          // staging buffers per lane quarter
template <int KIND, int TN, int RT, bool TA = false, bool SK = false>
struct Cfg {
    static constexpr bool I8 = KIND == KIND_I8;
    static constexpr bool WG = KIND == KIND_WGRAD;      // dense bf16 weight gradient: both operands by TMA, MN-major
    static constexpr bool W4 = !I8 && !WG;
    static_assert(!TA || (W4 && RT == 1), "tensor-memory A operand: A16W4 kinds, one row tile per CTA");
    static constexpr int A_BYTES = TA ? 0 : RT * A_TILE_BYTES;
    static constexpr int B_TILE_BYTES = TN * ROW_BYTES;
    static constexpr int RAW_TOTAL = W4 ? RT * RAW_BYTES : 0;
    static constexpr int STAGE_BYTES = A_BYTES + B_TILE_BYTES + RAW_TOTAL;
    static constexpr int FIX_BYTES = SK ? 4 * FIX_RING * FIX_COPY_BYTES : 0;    // balanced mode: the staging rings
    static constexpr int STAGES_FIT = (227 * 1024 - 1024 - 1024 - FIX_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_FIT > MAX_STAGES ? MAX_STAGES : STAGES_FIT;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + FIX_BYTES + 1024 /*alignment slack*/ + 1024 /*barriers*/;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static constexpr int ACC_COLS = RT * TN;                               // TMEM columns of one accumulator set
    static constexpr int TA_COLS = TA ? STAGES * TA_COLS_PER_STAGE : 0;    // one A slot per pipeline stage
    static constexpr int ACC_BUFS = (2 * ACC_COLS + TA_COLS <= 512) ? 2 : 1;   // double-buffered when TMEM allows
    static constexpr int TA_COL0 = ACC_BUFS * ACC_COLS;
    static constexpr int TMEM_NEED = ACC_BUFS * ACC_COLS + TA_COLS;
    static constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
    // Epilogue warps: one per TMEM lane quarter, or two (the second set behind all other warps, each warp of a pair
    // draining half of the token columns) where the accumulator is wide enough to split.  With a single accumulator
    // buffer the epilogue is exposed time between two tiles; splitting it halves that.
    static constexpr int EPI_SPLIT = (!SK && TN >= 64) ? 2 : 1;
    static constexpr int FIRST_EXTRA_EPI = 6 + (W4 ? NUM_DQ_WARPS : 0);
    static constexpr int NUM_WARPS = FIRST_EXTRA_EPI + (EPI_SPLIT - 1) * 4;
    static constexpr int THREADS = NUM_WARPS * 32;
    static constexpr uint32_t TX_BYTES = (uint32_t)(B_TILE_BYTES + (W4 ? RAW_TOTAL : A_BYTES));
    static constexpr int UMMA_PER_STAGE = 4;   // 128 bytes of contraction per stage / 32 bytes per MMA
    static_assert(TMEM_NEED <= 512 && STAGES >= 2, "tile configuration does not fit");
    static_assert(!W4 || STAGES >= 4, "the four dequant teams need at least four pipeline stages");
};

struct SmemCtl {
    uint64_t full[MAX_STAGES];     // TMA landed
    uint64_t a_ready[MAX_STAGES];  // dequantised tile written
    uint64_t empty[MAX_STAGES];    // MMAs that read the stage retired
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t fix_full[4][FIX_RING];   // balanced mode: hand-over copy landed (per lane quarter, per staging buffer)
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(SmemCtl) <= 1024, "barrier block of the shared-memory budget");

// ---------------------------------------------------------------------------------------------
// int4 -> bf16 dequant of 8 codes held in one little-endian 32-bit word of the nibble-pair layout
// (byte j = code[2j] << 4 | code[2j+1]).  q+128 is formed exactly by OR-ing the nibble into the mantissa
// of bf16 128.0; (q+128)-(z+128) and the product with s are single bf16 roundings, i.e. exactly
// bf16((q - z) * s) as DeQfunc_4bit_g computes it with bf16 qparams.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf2_as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 u32_as_bf2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }
// (w & 0x000F000F) | 0x43004300 as ONE three-input logic instruction (spelled out: the C expression compiled to more)
__device__ __forceinline__ uint32_t lop_nib(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint4 dequant8(uint32_t w, __nv_bfloat162 z128, __nv_bfloat162 s2) {
    const uint32_t p15 = lop_nib(w);             // (c1, c5)
    const uint32_t p04 = lop_nib(w >> 4);        // (c0, c4)
    const uint32_t p37 = lop_nib(w >> 8);        // (c3, c7)
    const uint32_t p26 = lop_nib(w >> 12);       // (c2, c6)
    uint32_t d15 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p15), z128), s2));
    uint32_t d04 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p04), z128), s2));
    uint32_t d37 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p37), z128), s2));
    uint32_t d26 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p26), z128), s2));
    uint4 o;
    o.x = __byte_perm(d04, d15, 0x5410);   // (c0, c1)
    o.y = __byte_perm(d26, d37, 0x5410);   // (c2, c3)
    o.z = __byte_perm(d04, d15, 0x7632);   // (c4, c5)
    o.w = __byte_perm(d26, d37, 0x7632);   // (c6, c7)
    return o;
}

// The same with a scale and a zero point of its own for every code: sp / zp hold (s, z + 128) of the pairs
// (c0,c4) (c1,c5) (c2,c6) (c3,c7) in x, y, z, w - the order the extraction produces.
__device__ __forceinline__ uint4 dequant8t(uint32_t w, const uint4& zp, const uint4& sp) {
    const uint32_t p15 = lop_nib(w);             // (c1, c5)
    const uint32_t p04 = lop_nib(w >> 4);        // (c0, c4)
    const uint32_t p37 = lop_nib(w >> 8);        // (c3, c7)
    const uint32_t p26 = lop_nib(w >> 12);       // (c2, c6)
    uint32_t d15 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p15), u32_as_bf2(zp.y)), u32_as_bf2(sp.y)));
    uint32_t d04 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p04), u32_as_bf2(zp.x)), u32_as_bf2(sp.x)));
    uint32_t d37 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p37), u32_as_bf2(zp.w)), u32_as_bf2(sp.w)));
    uint32_t d26 = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(p26), u32_as_bf2(zp.z)), u32_as_bf2(sp.z)));
    uint4 o;
    o.x = __byte_perm(d04, d15, 0x5410);   // (c0, c1)
    o.y = __byte_perm(d26, d37, 0x5410);   // (c2, c3)
    o.z = __byte_perm(d04, d15, 0x7632);   // (c4, c5)
    o.w = __byte_perm(d26, d37, 0x7632);   // (c6, c7)
    return o;
}

// ---------------------------------------------------------------------------------------------
// Transposed copy of a packed A16W4 weight for the grad-input GEMM.
//   dx[M,K] = dy[M,N] . W[N,K] contracts over the weight's ROWS.  With the weight as stored, the tensor-memory
//   placement of the dequantised tile would need a nibble-wise gather over 64 rows per thread, and the
//   shared-memory placement is bound by the shared-memory port (171 instead of 138 cycles per MMA).  With a
//   transposed copy Wt[K, N] (codes packed along n) the grad-input IS the forward kernel: dx = dy . Wt^T.  Scales
//   and zero points then differ per contraction element (they belong to (n, k / group)), so they are laid out
//   per (k group, 8 n) in exactly the order dequant8t consumes: 32 bytes = (s04 s15 s26 s37)(z04 z15 z26 z37), z
//   already offset by 128.  Both kernels run once per grad-input call (the weights may have changed since the last).
// ---------------------------------------------------------------------------------------------
// One CTA transposes a tile of 64 n x 256 k: codes go to shared memory as words of four consecutive k (one byte per
// code), a thread then owns four k and sixteen n: (even n << 4 | odd n) byte-wise gives the packed output bytes of all
// four k at once, three byte permutes per output word sort them into the four rows it writes (8 bytes each; the four
// threads of a k share a 32-byte segment).
__global__ void __launch_bounds__(256) k_w4_transpose(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int N, int K) {
    __shared__ uint32_t t[64][65];                        // [n][k / 4], one word of padding
    const int n0 = blockIdx.y * 64, k0 = blockIdx.x * 256, i = threadIdx.x;
    {
        const int n = i >> 2, seg = i & 3;                // 32 bytes = 64 codes of row n0 + n, k = k0 + seg * 64 ..
        const uint4* src = reinterpret_cast<const uint4*>(in + (size_t)(n0 + n) * (K / 2) + (k0 / 2) + seg * 32);
        const uint4 v0 = src[0], v1 = src[1];
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int h = 0; h < 8; ++h) {                     // byte j of the word: codes 2j (high nibble), 2j + 1 (low)
            const uint32_t hi = (w[h] >> 4) & 0x0F0F0F0Fu, lo = w[h] & 0x0F0F0F0Fu;
            t[n][seg * 16 + h * 2 + 0] = __byte_perm(hi, lo, 0x5140);      // c0 c1 c2 c3 = hi.b0 lo.b0 hi.b1 lo.b1
            t[n][seg * 16 + h * 2 + 1] = __byte_perm(hi, lo, 0x7362);      // c4 c5 c6 c7
        }
    }
    __syncthreads();
    {
        const int k4 = i >> 2, seg = i & 3;               // k = k0 + 4 k4 .. + 3, n = n0 + seg * 16 ..
        uint32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (t[seg * 16 + 2 * j][k4] << 4) | t[seg * 16 + 2 * j + 1][k4];
        const uint32_t a01 = __byte_perm(v[0], v[1], 0x5140), b01 = __byte_perm(v[0], v[1], 0x7362);   // bytes (k0 k0 k1 k1) / (k2 k2 k3 k3) of v0, v1
        const uint32_t a23 = __byte_perm(v[2], v[3], 0x5140), b23 = __byte_perm(v[2], v[3], 0x7362);
        const uint32_t a45 = __byte_perm(v[4], v[5], 0x5140), b45 = __byte_perm(v[4], v[5], 0x7362);
        const uint32_t a67 = __byte_perm(v[6], v[7], 0x5140), b67 = __byte_perm(v[6], v[7], 0x7362);
        uint8_t* dst = out + (size_t)(k0 + 4 * k4) * (N / 2) + (n0 / 2) + seg * 8;
        const size_t pitch = (size_t)(N / 2);
        *reinterpret_cast<uint2*>(dst) = make_uint2(__byte_perm(a01, a23, 0x5410), __byte_perm(a45, a67, 0x5410));
        *reinterpret_cast<uint2*>(dst + pitch) = make_uint2(__byte_perm(a01, a23, 0x7632), __byte_perm(a45, a67, 0x7632));
        *reinterpret_cast<uint2*>(dst + 2 * pitch) = make_uint2(__byte_perm(b01, b23, 0x5410), __byte_perm(b45, b67, 0x5410));
        *reinterpret_cast<uint2*>(dst + 3 * pitch) = make_uint2(__byte_perm(b01, b23, 0x7632), __byte_perm(b45, b67, 0x7632));
    }
}
// one thread per (8 n, k group); consecutive threads take consecutive groups, so the 2-byte reads of a warp are contiguous
__global__ void __launch_bounds__(256) k_w4_qp_transpose(const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ zeros,
                                                         uint4* __restrict__ qpt, int N, int G) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= G * (N / 8)) return;
    const int n8 = idx / G, g = idx - n8 * G, n = n8 * 8;
    const unsigned short* sp = reinterpret_cast<const unsigned short*>(scales);
    uint32_t sv[8], zv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        sv[j] = sp[(size_t)(n + j) * G + g];
        const __nv_bfloat16 z = __hadd(zeros[(size_t)(n + j) * G + g], __float2bfloat16_rn(128.0f));
        zv[j] = *reinterpret_cast<const unsigned short*>(&z);
    }
    uint4* dst = qpt + ((size_t)g * (size_t)(N / 8) + (size_t)n8) * 2;
    dst[0] = make_uint4(sv[0] | sv[4] << 16, sv[1] | sv[5] << 16, sv[2] | sv[6] << 16, sv[3] | sv[7] << 16);
    dst[1] = make_uint4(zv[0] | zv[4] << 16, zv[1] | zv[5] << 16, zv[2] | zv[6] << 16, zv[3] | zv[7] << 16);
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int KIND, int TN, int RT, bool TA, bool SK, bool QPT = false>
__global__ void __launch_bounds__(Cfg<KIND, TN, RT, TA, SK>::THREADS, 1)
k_gemm(const __grid_constant__ CUtensorMap map_tok, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
    static_assert(!SK || (KIND != KIND_I8 && RT == 1 && TN % FIX_COLS == 0), "balanced mode: A16W4 kinds, one row tile per CTA");
    static_assert(!QPT || (KIND == KIND_FWD && TA && RT == 1), "per-column group parameters: forward kernel, weight tile in tensor memory");
    using C = Cfg<KIND, TN, RT, TA, SK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem + C::STAGES * C::STAGE_BYTES + C::FIX_BYTES);
    volatile int* abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = smem_u32(smem);
    // stage layout: [A tile 0 .. RT-1][B tile][raw 0 .. RT-1]
    auto a_tile = [&](int s, int r) { return smem_base + s * C::STAGE_BYTES + r * A_TILE_BYTES; };
    auto b_tile = [&](int s) { return smem_base + s * C::STAGE_BYTES + C::A_BYTES; };
    auto raw_tile = [&](int s, int r) { return smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_TILE_BYTES + r * RAW_BYTES; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->a_ready[s]), 4);   // the 4 warps of the team that converts the stage
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->acc_full[a]), 1);
            mbar_init(smem_u32(&ctl->acc_empty[a]), 4 * C::EPI_SPLIT);
        }
        for (int q = 0; q < 4; ++q)
            for (int b = 0; b < FIX_RING; ++b) mbar_init(smem_u32(&ctl->fix_full[q][b]), 1);
        ctl->abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&ctl->tmem_base), C::TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) { tma_prefetch_desc(&map_tok); tma_prefetch_desc(&map_w); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    const bool prof = g_gemm_prof_on != 0;


    if (warp == 0) {
        // ===================== TMA producer =====================
        // warp-uniform loop, one elected lane issues the copies (same reason as for the MMA issuer below)
        {
            const bool leader = elect_one_sync();
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            long long w_empty = 0;
            SegWalk<SK> walk(p);
            Seg sg;
            while (ok && walk.next(p, sg)) {
                const int r_tile = sg.r_tile, t_tile = sg.t_tile;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
                    if (!(ok = mbar_wait_t(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, prof, w_empty))) break;
                    const uint32_t bar = smem_u32(&ctl->full[stage]);
                    if (leader) {
                        mbar_expect_tx(bar, C::TX_BYTES);
#pragma unroll
                        for (int r = 0; r < RT; ++r) {
                            const int row0 = (r_tile * RT + r) * TILE_R;
                            if (KIND == KIND_I8)            // int8 weights straight into the MMA tile
                                tma_load_2d(a_tile(stage, r), &map_w, kb * 128, row0, bar);
                            else if (KIND == KIND_WGRAD) {  // dY[64 tokens, 128 n] as two MN-major atoms of 64 n (128 B rows)
                                tma_load_2d(a_tile(stage, r), &map_w, row0, kb * 64, bar);
                                tma_load_2d(a_tile(stage, r) + 8192u, &map_w, row0 + 64, kb * 64, bar);
                            } else if (KIND == KIND_FWD)    // raw: 128 weight rows x 32 bytes (64 k)
                                tma_load_2d(smem_u32(raw_tile(stage, r)), &map_w, kb * 32, row0, bar);
                            else                            // raw: 64 weight rows (n) x 64 bytes (128 k)
                                tma_load_2d(smem_u32(raw_tile(stage, r)), &map_w, row0 / 2, kb * 64, bar);
                        }
                        if (KIND == KIND_WGRAD) {           // X[64 tokens, TN k] as TN/64 MN-major atoms
#pragma unroll
                            for (int h = 0; h < TN / 64; ++h)
                                tma_load_2d(b_tile(stage) + (uint32_t)(h * 8192), &map_tok, t_tile * TN + h * 64, kb * 64, bar);
                        } else {
                            tma_load_2d(b_tile(stage), &map_tok, kb * (C::I8 ? 128 : 64), t_tile * TN, bar);
                        }
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (prof && lane == 0) atomicAdd(&g_gemm_prof[0], (unsigned long long)w_empty);
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        // The whole warp walks the loop and one elected lane issues the MMAs and commits.  With the loop inside an
        // `if (lane == 0)` the operands of every tcgen05.mma are per-thread values and the issuing thread's own
        // instruction latencies bound the kernel at token tiles of 128 and below (a stage of four MMAs took ~480
        // cycles to issue against 256 cycles of tensor work); kept warp-uniform they cost ~290.
        // No warp-level synchronisation sits inside the loop: if a bounded wait gives up in some lanes only, those lanes
        // leave for the teardown and the others follow at their next wait (the abort flag is raised).
        {
            constexpr uint32_t IDESC = make_idesc(C::I8, (KIND == KIND_DGRAD && !TA) || C::WG, TN, C::WG);
            const bool leader = elect_one_sync();
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            long long w_full = 0, w_aready = 0, w_acc = 0;
            const long long t_role = prof ? clock64() : 0;
            SegWalk<SK> walk(p);
            Seg sg;
            while (ok && walk.next(p, sg)) {
                const int kb0 = sg.kb0, kb1 = sg.kb1;
                if (!(ok = mbar_wait_t(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort_flag, prof, w_acc))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * C::ACC_COLS);
                for (int kb = kb0; kb < kb1; ++kb) {
                    // A16W4: the team that converted the stage waited for its TMA data before it started, so its
                    // `a_ready` arrival also covers the token tile: one barrier round trip per stage instead of two
                    if (C::W4) { if (!(ok = mbar_wait_t(smem_u32(&ctl->a_ready[stage]), phase, abort_flag, prof, w_aready))) break; }
                    else { if (!(ok = mbar_wait_t(smem_u32(&ctl->full[stage]), phase, abort_flag, prof, w_full))) break; }
                    tc_fence_after();
                    // K-major tiles: 8-row groups are 1024 B apart; one MMA consumes 32 B of every row.
                    // MN-major A (grad-input): 64-element atoms are 8192 B apart (leading), 8-row groups of the
                    // contraction 1024 B apart (stride); one MMA consumes 16 contraction rows = 2048 B.
                    const uint64_t b_desc = C::WG ? make_smem_desc(b_tile(stage), 8192, 1024) : make_smem_desc(b_tile(stage), 16, 1024);
                    const uint32_t a_step = (KIND == KIND_DGRAD || C::WG) ? (2048u >> 4) : (32u >> 4);
                    const uint32_t b_step = C::WG ? (2048u >> 4) : (32u >> 4);
                    const uint32_t first = kb > kb0 ? 1u : 0u;
                    if (leader) {
                        if (TA) {
                            const uint32_t a_tmem = tmem_base + (uint32_t)(C::TA_COL0 + stage * TA_COLS_PER_STAGE);
#pragma unroll
                            for (int kk = 0; kk < C::UMMA_PER_STAGE; ++kk)
                                umma_ta(d_tmem, a_tmem + (uint32_t)(kk * 8), b_desc + (uint64_t)(kk * b_step), IDESC, kk > 0 ? 1u : first);
                        } else {
#pragma unroll
                            for (int r = 0; r < RT; ++r) {
                                const uint64_t a_desc = (KIND == KIND_DGRAD || C::WG) ? make_smem_desc(a_tile(stage, r), 8192, 1024)
                                                                                      : make_smem_desc(a_tile(stage, r), 16, 1024);
#pragma unroll
                                for (int kk = 0; kk < C::UMMA_PER_STAGE; ++kk)
                                    umma<C::I8>(d_tmem + (uint32_t)(r * TN), a_desc + (uint64_t)(kk * a_step), b_desc + (uint64_t)(kk * b_step),
                                                IDESC, kk > 0 ? 1u : first);
                            }
                        }
                        umma_commit(smem_u32(&ctl->empty[stage]));
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (leader) umma_commit(smem_u32(&ctl->acc_full[acc]));
                if (++acc == C::ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
            }
            if (prof && lane == 0) {
                atomicAdd(&g_gemm_prof[1], (unsigned long long)w_full); atomicAdd(&g_gemm_prof[2], (unsigned long long)w_aready);
                atomicAdd(&g_gemm_prof[3], (unsigned long long)w_acc); atomicAdd(&g_gemm_prof[4], (unsigned long long)(clock64() - t_role));
                atomicAdd(&g_gemm_prof[9], 1ull);
            }
        }
    } else if (warp < 6 || warp >= C::FIRST_EXTRA_EPI) {
        // ===================== epilogue =====================
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int col_lo = (warp < 6 ? 0 : 1) * (TN / C::EPI_SPLIT), col_hi = col_lo + TN / C::EPI_SPLIT;   // its token columns
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        long long w_accf = 0;
        const long long t_role = prof ? clock64() : 0;
        SegWalk<SK> walk(p);
        Seg sg;
        // Balanced mode.  A segment that covers part of a shared tile's k range publishes its fp32 partial sums in a slot
        // of the workspace ([shared tile][part][lane quarter][token column][32 rows]) and takes a ticket of the (tile,
        // lane quarter).  Whoever draws the last ticket adds the tile's parts up in k order (owner's head first, then the
        // helpers' pieces; always the same order, whoever does it) and runs the ordinary epilogue on the sums.  Nobody
        // waits for another CTA.  An owner first looks at the ticket counter: when every helper has already published
        // (the schedule is built for that), it skips its own publication and starts from its accumulator.  The other
        // parts come in as 2 KB bulk copies (16 token columns of one part) through a ring of staging buffers per lane
        // quarter, several copies ahead of the additions.
        float* const sk_slots = reinterpret_cast<float*>(p.partial);
        unsigned int* const sk_tickets = SK ? reinterpret_cast<unsigned int*>(sk_slots + (size_t)p.sk_rem * p.sk_pmax * (TN * TILE_R)) : nullptr;
        uint8_t* const fix_ring = smem + C::STAGES * C::STAGE_BYTES + quad * FIX_RING * FIX_COPY_BYTES;
        uint32_t fix_phase = 0;                    // bit b: parity to wait for on staging buffer b of this quarter
        while (ok && walk.next(p, sg)) {
            const int r_tile = sg.r_tile, t_tile = sg.t_tile, split = sg.split;
            if (!(ok = mbar_wait_t(smem_u32(&ctl->acc_full[acc]), acc_phase, abort_flag, prof, w_accf))) break;
            tc_fence_after();
            bool emit = true, sk_sum = false;
            int sk_parts = 1, sk_part_lo = 0;      // parts of the tile; first part that comes through the ring (1: own sums from the accumulator)
            int sk_issued = 0, sk_taken = 0, sk_copies = 0, sk_is = 0, sk_ip = 0;   // copies issued / consumed / in all; slab and part of the next issue
            const float* sk_part0 = nullptr;       // this quarter's share of the tile's first slot
            auto sk_issue = [&]() {                // next copy of the sequence (slab-major, parts in k order inside a slab)
                const float* src = sk_part0 + (size_t)sk_ip * 4 * (TN * 32) + (size_t)sk_is * (FIX_COLS * 32);
                if (lane == 0) {
                    const int b = sk_issued & (FIX_RING - 1);
                    const uint32_t bar = smem_u32(&ctl->fix_full[quad][b]);
                    mbar_expect_tx(bar, FIX_COPY_BYTES);
                    bulk_load(smem_u32(fix_ring + b * FIX_COPY_BYTES), src, FIX_COPY_BYTES, bar);
                }
                ++sk_issued;
                if (++sk_ip == sk_parts) { sk_ip = sk_part_lo; ++sk_is; }
            };
            if (SK && !(sg.kb0 == 0 && sg.kb1 == p.kb_total)) {
                const long long t_pub = prof ? clock64() : 0;
                const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C::ACC_COLS);
                const int j = t_tile * p.r_tiles + r_tile - p.sk_full;      // shared tile
                const int tail = p.kb_total - p.sk_h;
                const int h_first = sk_helper_of(p, j * tail), h_last = sk_helper_of(p, (j + 1) * tail - 1);
                sk_parts = 2 + h_last - h_first;
                const bool is_owner = sg.kb0 == 0;
                const int my_part = is_owner ? 0 : 1 + ((int)blockIdx.x - p.sk_rem) - h_first;
                sk_part0 = sk_slots + ((size_t)j * p.sk_pmax * 4 + (size_t)quad) * (size_t)(TN * 32);
                unsigned int* const ticket_ptr = sk_tickets + j * 4 + quad;
                unsigned int ticket = 0;
                if (is_owner) {                    // have all helpers published already?
                    if (lane == 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(ticket) : "l"(ticket_ptr) : "memory");
                    ticket = __shfl_sync(0xffffffffu, ticket, 0);
                }
                if (is_owner && ticket == (unsigned int)(sk_parts - 1)) {
                    sk_part_lo = 1;                // own sums stay in the accumulator
                } else {
                    // publish: lanes are consecutive rows, every store instruction writes 128 contiguous bytes
                    float* dst = const_cast<float*>(sk_part0) + (size_t)my_part * 4 * (TN * 32) + lane;
#pragma unroll 1
                    for (int c0 = 0; c0 < TN; c0 += 16) {
                        uint32_t v[16];
                        tmem_ld16(acc_addr + (uint32_t)c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) dst[(c0 + jj) * 32] = __uint_as_float(v[jj]);
                    }
                    fence_proxy_async_all();       // the slot is read back with bulk copies (async proxy)
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) ticket = atomicAdd(ticket_ptr, 1u);
                    ticket = __shfl_sync(0xffffffffu, ticket, 0);
                }
                emit = sk_sum = ticket == (unsigned int)(sk_parts - 1);
                if (prof && warp == 2 && lane == 0) atomicAdd(&g_gemm_prof[10], (unsigned long long)(clock64() - t_pub));
                if (sk_sum) {
                    __threadfence();
                    fence_proxy_async_all();
                    sk_ip = sk_part_lo;
                    sk_copies = (sk_parts - sk_part_lo) * (TN / FIX_COLS);
                    for (int i = 0; i < FIX_RING && i < sk_copies; ++i) sk_issue();
                    if (prof && warp == 2 && lane == 0) { atomicAdd(&g_gemm_prof[12], 1ull); atomicAdd(&g_gemm_prof[14], (unsigned long long)sk_copies); }
                }
            }
            const long long t_emit = prof ? clock64() : 0;
            if (emit) {
#pragma unroll 1
            for (int rr = 0; rr < RT; ++rr) {
                const int r = (r_tile * RT + rr) * TILE_R + quad * 32 + lane;
                const bool r_ok = r < p.R;
                const float cs = (C::I8 && p.col_scale && r_ok) ? __ldg(p.col_scale + r) : 1.0f;
                const float bias = (p.bias && r_ok) ? __bfloat162float(p.bias[r]) : 0.0f;
                // tokens per TMEM read-out: the int8 kernel has registers to spare (6 warps) and halves the number of
                // load-wait round trips; the A16W4 kernels run at the register cap of a 22-warp CTA
                constexpr int SLAB = (C::I8 && TN >= 32) ? 32 : 16;
#pragma unroll 1
                for (int c0 = col_lo; c0 < col_hi; c0 += SLAB) {
                    uint32_t v[SLAB];
                    if (SK && sk_sum) {
                        // the slab's sums: the tile's parts in k order, each a 2 KB copy in the staging ring (the first
                        // from the accumulator when this is the owner and it did not publish)
                        if (sk_part_lo) {
                            tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C::ACC_COLS + c0), *reinterpret_cast<uint32_t(*)[16]>(&v[0]));
                            tmem_ld_wait();
                        }
#pragma unroll 1
                        for (int part = sk_part_lo; part < sk_parts; ++part) {
                            const int b = sk_taken & (FIX_RING - 1);
                            if (ok) ok = mbar_wait(smem_u32(&ctl->fix_full[quad][b]), (fix_phase >> b) & 1u, abort_flag);
                            fix_phase ^= 1u << b;
                            const float* src = reinterpret_cast<const float*>(fix_ring + b * FIX_COPY_BYTES) + lane;
                            if (part == 0) {
#pragma unroll
                                for (int jj = 0; jj < 16; ++jj) v[jj] = __float_as_uint(src[jj * 32]);
                            } else {
#pragma unroll
                                for (int jj = 0; jj < 16; ++jj) v[jj] = __float_as_uint(__fadd_rn(__uint_as_float(v[jj]), src[jj * 32]));
                            }
                            ++sk_taken;
                            __syncwarp();                                     // every lane has read the buffer: refill it
                            if (ok && sk_issued < sk_copies) sk_issue();
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < SLAB / 16; ++h)
                            tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C::ACC_COLS + rr * TN + c0 + 16 * h),
                                      *reinterpret_cast<uint32_t(*)[16]>(&v[16 * h]));
                        tmem_ld_wait();
                    }
                    if (C::WG) {
                        // weight gradient: lane = output row n, the slab's 16 columns are consecutive in memory.
                        // dW = bf16(fp32(dW) + acc) when accumulating (what a GEMM with beta = 1 computes), else bf16(acc).
                        const int t0 = t_tile * TN + c0;
                        if (r_ok && t0 < p.M) {
                            __nv_bfloat16* dst = p.out + (size_t)r * p.M + t0;
                            if (t0 + SLAB <= p.M && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                                uint4 o[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                                if (p.accumulate) { o[0] = *reinterpret_cast<const uint4*>(dst); o[1] = *reinterpret_cast<const uint4*>(dst + 8); }
                                uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const float a0 = __fadd_rn(__uint_as_float(ow[i] << 16), __uint_as_float(v[2 * i]));
                                    const float a1 = __fadd_rn(__uint_as_float(ow[i] & 0xffff0000u), __uint_as_float(v[2 * i + 1]));
                                    ow[i] = bf2_as_u32(__floats2bfloat162_rn(a0, a1));
                                }
                                *reinterpret_cast<uint4*>(dst) = o[0]; *reinterpret_cast<uint4*>(dst + 8) = o[1];
                            } else {
#pragma unroll
                                for (int j = 0; j < SLAB; ++j) {
                                    if (t0 + j >= p.M) break;
                                    const float old = p.accumulate ? __bfloat162float(dst[j]) : 0.0f;
                                    dst[j] = __float2bfloat16_rn(__fadd_rn(old, __uint_as_float(v[j])));
                                }
                            }
                        }
                        continue;
                    }
                    if (p.splits == 1 && !(C::I8 && p.acc_out) && t_tile * TN + c0 + SLAB <= p.M &&
                        (!C::I8 || (reinterpret_cast<uintptr_t>(p.row_scale) & 15) == 0)) {       // warp-uniform condition
                        // Full slab of SLAB tokens.  Two results per conversion instruction (the single-value conversion
                        // issues on the slow pipe); pk[i] = bf16 results of tokens (2i, 2i+1) for this lane's row.
                        const int t0 = t_tile * TN + c0;
                        uint32_t pk[SLAB / 2];
                        if (C::W4) {
#pragma unroll
                            for (int i = 0; i < SLAB / 2; ++i) {
                                pk[i] = bf2_as_u32(__floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])));
                                if (p.bias)         // mm output is rounded to bf16 first, the bias is added after
                                    pk[i] = bf2_as_u32(__floats2bfloat162_rn(__fadd_rn(__uint_as_float(pk[i] << 16), bias),
                                                                             __fadd_rn(__uint_as_float(pk[i] & 0xffff0000u), bias)));
                            }
                        } else {
                            // acc * row_scale[t] * col_scale[r] * alpha + bias; the 16 token scales are the same addresses
                            // for every lane: four broadcast 16-byte loads
                            float rs[SLAB];
                            if (p.row_scale) {
                                const float4* rp = reinterpret_cast<const float4*>(p.row_scale + t0);
#pragma unroll
                                for (int q = 0; q < SLAB / 4; ++q) { const float4 t4 = __ldg(rp + q); rs[4 * q] = t4.x; rs[4 * q + 1] = t4.y; rs[4 * q + 2] = t4.z; rs[4 * q + 3] = t4.w; }
                            } else {
#pragma unroll
                                for (int j = 0; j < SLAB; ++j) rs[j] = 1.0f;
                            }
#pragma unroll
                            for (int i = 0; i < SLAB / 2; ++i) {
                                float f0 = (float)(int32_t)v[2 * i], f1 = (float)(int32_t)v[2 * i + 1];
                                if (p.row_scale) { f0 = __fmul_rn(f0, rs[2 * i]); f1 = __fmul_rn(f1, rs[2 * i + 1]); }
                                f0 = __fadd_rn(__fmul_rn(__fmul_rn(f0, cs), p.alpha), bias);
                                f1 = __fadd_rn(__fmul_rn(__fmul_rn(f1, cs), p.alpha), bias);
                                pk[i] = bf2_as_u32(__floats2bfloat162_rn(f0, f1));
                            }
                        }
                        // (a transpose through shared memory into 16-byte stores was tried: slower than these 2-byte stores)
                        if (r_ok) {
                            unsigned short* o16 = reinterpret_cast<unsigned short*>(p.out + (size_t)t0 * p.R + r);
                            const size_t stride = (size_t)p.R;
#pragma unroll
                            for (int i = 0; i < SLAB / 2; ++i) {
                                o16[(2 * i) * stride] = (unsigned short)(pk[i] & 0xffffu);
                                o16[(2 * i + 1) * stride] = (unsigned short)(pk[i] >> 16);
                            }
                        }
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < SLAB; ++j) {
                        const int t = t_tile * TN + c0 + j;
                        if (!r_ok || t >= p.M) continue;
                        const size_t o = (size_t)t * p.R + r;
                        if (p.splits > 1) {
                            reinterpret_cast<uint32_t*>(p.partial)[(size_t)split * p.M * p.R + o] = v[j];
                        } else if (C::I8) {
                            const int32_t a = (int32_t)v[j];
                            if (p.acc_out) p.acc_out[o] = a;
                            float f = (float)a;
                            if (p.row_scale) f = __fmul_rn(f, __ldg(p.row_scale + t));
                            f = __fmul_rn(__fmul_rn(f, cs), p.alpha);
                            p.out[o] = __float2bfloat16_rn(__fadd_rn(f, bias));
                        } else {
                            float f = bf16r(__uint_as_float(v[j]));          // mm output is bf16, bias added after
                            p.out[o] = __float2bfloat16_rn(p.bias ? __fadd_rn(f, bias) : f);
                        }
                    }
                }
            }
            }   // emit
            if (SK && sk_sum && prof && warp == 2 && lane == 0) atomicAdd(&g_gemm_prof[11], (unsigned long long)(clock64() - t_emit));
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
            if (++acc == C::ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
        }
        if (prof && warp == 2 && lane == 0) {
            atomicAdd(&g_gemm_prof[7], (unsigned long long)w_accf); atomicAdd(&g_gemm_prof[8], (unsigned long long)(clock64() - t_role));
        }
    } else {
        // ===================== dequant (A16W4) =====================
        if (C::W4 && warp < 6 + NUM_DQ_WARPS) {
            // The 16 warps form 4 teams of 4 warps; team g converts pipeline stages g, g+4, g+8, ... on its own, which
            // keeps four stages of conversion in flight (one stage is a dependent chain: shared-memory loads, ALU work,
            // the store of the tile and its completion fence).
            //
            // Tensor-memory A operand (TA): a warp may only write the TMEM lane quarter (warp id % 4); every team has
            // one warp per quarter.
            //   forward   : lane = weight row, the stage's 64 k -> 32 columns of that lane
            //   grad-input: lane = k inside the 128-tile, the stage's 64 weight rows n -> 32 columns (two n per column);
            //               lane j fetches scale / zero point of rows n_j and n_j+32, shared by shuffle
            // Shared-memory A operand: thread tt of the team owns 32 raw bytes = 64 weights of one weight row and
            // writes them as eight 16-byte chunks of the 128-byte-swizzled tile.
            //   forward   : raw [128 rows][32 B]; row = tt                 -> row tt of the K-major tile
            //   grad-input: raw [ 64 rows][64 B]; row = tt/2, half = tt%2  -> row tt/2 of MN-atom `half`
            const int quarter = warp & 3, team = (warp - 6) >> 2;
            const int tt = ((warp - 6) & 3) * 32 + lane;
            const int groups_per_row = p.wcols / p.group;
            // k / group without a division in the per-stage path: groups are multiples of 32 and so is every k asked for
            const int g32 = p.group >> 5;
            const int g_shift = (g32 & (g32 - 1)) == 0 ? 31 - __clz(g32) : -1;
            auto group_of = [&](int k) { const int k32 = k >> 5; return g_shift >= 0 ? (k32 >> g_shift) : (k32 / g32); };
            const uint32_t ta_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)C::TA_COL0;
            // position in this CTA's sequence of k-blocks: the walker stands behind the segment that holds k-block `kb`
            struct Pos { SegWalk<SK> walk; int kb, kb1, r_tile; bool valid; };
            auto advance = [&](Pos& q, int n) {
                q.kb += n;
                while (q.valid && q.kb >= q.kb1) {
                    const int over = q.kb - q.kb1;
                    Seg sg;
                    if (!q.walk.next(p, sg)) { q.valid = false; break; }
                    q.kb = sg.kb0 + over; q.kb1 = sg.kb1; q.r_tile = sg.r_tile;
                }
            };
            // (scale | zero << 16) as raw bf16 bits for this thread's two 32-element slots of row tile r at position q
            auto load_qp2 = [&](const Pos& q, int r, uint32_t& a, uint32_t& b) {
                a = b = 0u;
                if (QPT || !q.valid) return;
                int wrow, k0, k1;
                if (TA && KIND == KIND_DGRAD) {            // rows n_lane and n_lane+32, one k group per warp
                    wrow = q.kb * 64 + lane; k0 = k1 = q.r_tile * TILE_R + quarter * 32;
                } else if (KIND == KIND_FWD) {
                    wrow = (q.r_tile * RT + r) * TILE_R + (TA ? quarter * 32 + lane : tt); k0 = q.kb * 64; k1 = k0 + 32;
                } else {
                    wrow = q.kb * 64 + (tt >> 1); k0 = (q.r_tile * RT + r) * TILE_R + (tt & 1) * 64; k1 = k0 + 32;
                }
                const int n_rows = (KIND == KIND_FWD) ? p.R : p.C;
                if (wrow >= n_rows || k0 >= p.wcols) return;
                const int gk0 = group_of(k0);
                const size_t g0 = (size_t)wrow * groups_per_row + (size_t)gk0;
                const size_t g1 = (TA && KIND == KIND_DGRAD) ? g0 + (size_t)32 * groups_per_row : g0 + (size_t)(group_of(k1) - gk0);
                const unsigned short* sp = reinterpret_cast<const unsigned short*>(p.scales);
                const unsigned short* zp = reinterpret_cast<const unsigned short*>(p.zeros);
                a = (uint32_t)__ldg(sp + g0) | ((uint32_t)__ldg(zp + g0) << 16);
                b = a;
                if (g1 != g0) b = (uint32_t)__ldg(sp + g1) | ((uint32_t)__ldg(zp + g1) << 16);   // groups of 64 and up: one pair per thread
            };
            constexpr int PF = 2;                                          // own stages of qparam prefetch
            Pos cur{SegWalk<SK>(p), 0, 0, 0, true};
            advance(cur, 0);                                               // opens the first segment (kb == kb1 == 0)
            advance(cur, team);
            Pos pre = cur;
            uint32_t qa[PF][RT], qb[PF][RT];
#pragma unroll
            for (int u = 0; u < PF; ++u) {
#pragma unroll
                for (int r = 0; r < RT; ++r) load_qp2(pre, r, qa[u][r], qb[u][r]);
                advance(pre, 4);
            }
            uint32_t cnt = (uint32_t)team;
            bool ok = true;
            long long w_dq = 0;
            const long long t_role = prof ? clock64() : 0;
            const __nv_bfloat162 c128 = __float2bfloat162_rn(128.0f);
            while (ok && cur.valid) {
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    if (!cur.valid) break;
                    uint32_t ca[RT], cb[RT];
#pragma unroll
                    for (int r = 0; r < RT; ++r) { ca[r] = qa[u][r]; cb[r] = qb[u][r]; load_qp2(pre, r, qa[u][r], qb[u][r]); }
                    advance(pre, 4);
                    const int stage = (int)(cnt % (uint32_t)C::STAGES);
                    const uint32_t phase = (cnt / (uint32_t)C::STAGES) & 1u;
                    // This team did not take part in the stage's previous use (another team converted it), so it first
                    // waits, like the producer, until that use has been consumed; only then is the parity of the `full`
                    // wait unambiguous.  (Needs STAGES >= number of teams: then the stage's use before the previous one
                    // is known to be over, because the producer had to see it retired before it could fill this team's
                    // own previous stage.)
                    // With a stage count that is a multiple of the four teams a team meets the same stages every round
                    // and needs no such wait: `full` completing already implies that the producer saw the stage retired.
                    ok = (C::STAGES % 4 == 0 || mbar_wait_t(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, prof, w_dq)) &&
                         mbar_wait_t(smem_u32(&ctl->full[stage]), phase, abort_flag, prof, w_dq);
                    ok = __all_sync(0xffffffffu, ok) != 0;                 // the TMEM store below is warp-collective
                    if (!ok) break;
                    if (TA && KIND == KIND_DGRAD) {
                        const uint32_t dst = ta_addr + (uint32_t)(stage * TA_COLS_PER_STAGE);
                        const int kk = quarter * 32 + lane;
                        const uint8_t* rp = raw_tile(stage, 0) + (kk >> 1);
                        const uint32_t sh = (kk & 1) ? 0u : 4u;            // even k sits in the high nibble
#pragma unroll
                        for (int c8 = 0; c8 < 4; ++c8) {
                            uint32_t col[8];
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) {
                                const int n = (c8 * 8 + jj) * 2;           // weight rows n, n+1 of the stage
                                const uint32_t b0 = rp[n * 64], b1 = rp[(n + 1) * 64];
                                const uint32_t q2 = ((b0 >> sh) & 15u) | (((b1 >> sh) & 15u) << 16) | 0x43004300u;
                                const uint32_t src = (n < 32) ? ca[0] : cb[0];
                                const uint32_t qp0 = __shfl_sync(0xffffffffu, src, n & 31), qp1 = __shfl_sync(0xffffffffu, src, (n + 1) & 31);
                                const __nv_bfloat162 s2 = u32_as_bf2(__byte_perm(qp0, qp1, 0x5410));
                                const __nv_bfloat162 z128 = __hadd2_rn(u32_as_bf2(__byte_perm(qp0, qp1, 0x7632)), c128);
                                col[jj] = bf2_as_u32(__hmul2_rn(__hsub2_rn(u32_as_bf2(q2), z128), s2));
                            }
                            tmem_st8(dst + (uint32_t)(c8 * 8), make_uint4(col[0], col[1], col[2], col[3]), make_uint4(col[4], col[5], col[6], col[7]));
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < RT; ++r) {
                            const __nv_bfloat162 s2a = u32_as_bf2(__byte_perm(ca[r], ca[r], 0x1010)), s2b = u32_as_bf2(__byte_perm(cb[r], cb[r], 0x1010));
                            const __nv_bfloat162 za = __hadd2_rn(u32_as_bf2(__byte_perm(ca[r], ca[r], 0x3232)), c128);
                            const __nv_bfloat162 zb = __hadd2_rn(u32_as_bf2(__byte_perm(cb[r], cb[r], 0x3232)), c128);
                            const int raw_off = TA ? (quarter * 32 + lane) * 32 : tt * 32;   // dgrad: (tt/2)*64 + (tt%2)*32 == tt*32
                            const uint4* rp = reinterpret_cast<const uint4*>(raw_tile(stage, r) + raw_off);
                            const uint4 r0 = rp[0], r1 = rp[1];
                            if (TA && QPT) {
                                // group parameters of the stage's 64 contraction elements (the same for every row of the
                                // tile's k group: the loads of a warp are one broadcast each), one word ahead of their use
                                const uint32_t dst = ta_addr + (uint32_t)(stage * TA_COLS_PER_STAGE);
                                const uint4* qp = p.qpt + ((size_t)cur.r_tile * (size_t)(p.C >> 3) + (size_t)cur.kb * 8) * 2;
                                const uint32_t wq[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
                                uint4 sp = __ldg(qp), zp = __ldg(qp + 1);
#pragma unroll
                                for (int i = 0; i < 8; i += 2) {
                                    const uint4 sp1 = __ldg(qp + 2 * i + 2), zp1 = __ldg(qp + 2 * i + 3);
                                    const uint4 d0 = dequant8t(wq[i], zp, sp);
                                    if (i + 2 < 8) { sp = __ldg(qp + 2 * i + 4); zp = __ldg(qp + 2 * i + 5); }
                                    tmem_st8(dst + (uint32_t)(4 * i), d0, dequant8t(wq[i + 1], zp1, sp1));
                                }
                            } else if (TA) {
                                const uint32_t dst = ta_addr + (uint32_t)(stage * TA_COLS_PER_STAGE);
                                tmem_st8(dst + 0, dequant8(r0.x, za, s2a), dequant8(r0.y, za, s2a));
                                tmem_st8(dst + 8, dequant8(r0.z, za, s2a), dequant8(r0.w, za, s2a));
                                tmem_st8(dst + 16, dequant8(r1.x, zb, s2b), dequant8(r1.y, zb, s2b));
                                tmem_st8(dst + 24, dequant8(r1.z, zb, s2b), dequant8(r1.w, zb, s2b));
                            } else {
                                const int row = (KIND == KIND_FWD) ? tt : (tt >> 1);
                                const int atom = (KIND == KIND_FWD) ? 0 : (tt & 1);
                                uint8_t* dst = smem + stage * C::STAGE_BYTES + r * A_TILE_BYTES + atom * 8192 + row * ROW_BYTES;
                                const int swz = row & 7;
                                *reinterpret_cast<uint4*>(dst + ((0 ^ swz) << 4)) = dequant8(r0.x, za, s2a);
                                *reinterpret_cast<uint4*>(dst + ((1 ^ swz) << 4)) = dequant8(r0.y, za, s2a);
                                *reinterpret_cast<uint4*>(dst + ((2 ^ swz) << 4)) = dequant8(r0.z, za, s2a);
                                *reinterpret_cast<uint4*>(dst + ((3 ^ swz) << 4)) = dequant8(r0.w, za, s2a);
                                *reinterpret_cast<uint4*>(dst + ((4 ^ swz) << 4)) = dequant8(r1.x, zb, s2b);
                                *reinterpret_cast<uint4*>(dst + ((5 ^ swz) << 4)) = dequant8(r1.y, zb, s2b);
                                *reinterpret_cast<uint4*>(dst + ((6 ^ swz) << 4)) = dequant8(r1.z, zb, s2b);
                                *reinterpret_cast<uint4*>(dst + ((7 ^ swz) << 4)) = dequant8(r1.w, zb, s2b);
                            }
                        }
                    }
                    if (TA) { tmem_st_wait(); tc_fence_before(); } else { fence_proxy_async(); }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctl->a_ready[stage]));
                    cnt += 4u;
                    advance(cur, 4);
                }
            }
            if (prof && warp == 6 && lane == 0) {
                atomicAdd(&g_gemm_prof[5], (unsigned long long)w_dq); atomicAdd(&g_gemm_prof[6], (unsigned long long)(clock64() - t_role));
            }
        }
    }

    // ===================== teardown =====================
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give bulk copies that may still be in flight time to land before the CTA's shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(&g_gemm_status, 1);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// split-K reduction
// ---------------------------------------------------------------------------------------------
template <bool I8>
__global__ void __launch_bounds__(256) k_splitk_reduce(const GemmParams p) {
    const int64_t total = (int64_t)p.M * p.R;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i % p.R);
        const int t = (int)(i / p.R);
        if (I8) {
            int32_t a = 0;
            for (int s = 0; s < p.splits; ++s) a += reinterpret_cast<const int32_t*>(p.partial)[(size_t)s * total + i];
            if (p.acc_out) p.acc_out[i] = a;
            float f = (float)a;
            if (p.row_scale) f = __fmul_rn(f, __ldg(p.row_scale + t));
            f = __fmul_rn(__fmul_rn(f, p.col_scale ? __ldg(p.col_scale + r) : 1.0f), p.alpha);
            p.out[i] = __float2bfloat16_rn(__fadd_rn(f, p.bias ? __bfloat162float(p.bias[r]) : 0.0f));
        } else {
            float a = 0.0f;
            for (int s = 0; s < p.splits; ++s) a = __fadd_rn(a, reinterpret_cast<const float*>(p.partial)[(size_t)s * total + i]);
            float f = bf16r(a);
            p.out[i] = __float2bfloat16_rn(p.bias ? __fadd_rn(f, __bfloat162float(p.bias[r])) : f);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Host side: plan, tensor maps, launch
// ---------------------------------------------------------------------------------------------
// Where the dequantised weight tile is staged for the tensor core.  Forward: tensor memory (each lane is a weight
// row, so a thread converts whole words and the MMA reads no A bytes from shared memory).  Grad-input: shared
// memory, described MN-major (a TMEM lane would be one k, forcing a nibble-wise gather that needs about twice the
// instructions; measured slower).  LQ_GEMM_A_OPERAND=smem|tmem forces one placement for both (A/B runs, tests);
// read at every launch.
static bool a_operand_in_tmem(int kind) {
    const char* e = getenv("LQ_GEMM_A_OPERAND");
    if (e && e[0] == 's') return false;
    if (e && e[0] == 't') return true;
    return kind == KIND_FWD;
}

struct Plan {
    int tn, rt, r_tiles, t_tiles, splits, kb_total, kb_per_split;
    bool skinny;
    bool sk;                                                    // balanced forward (see SegWalk)
    int sk_grid, sk_full, sk_rem, sk_h, sk_helpers, sk_pmax;
};

// Balanced forward: bytes of the partial-sum slots (sk_pmax per shared tile) and of the tickets behind them.
static size_t sk_slot_bytes(const Plan& pl) { return (size_t)pl.sk_rem * pl.sk_pmax * (size_t)pl.tn * TILE_R * 4; }
static size_t sk_ticket_bytes(const Plan& pl) { return (size_t)pl.sk_rem * 4 * sizeof(unsigned int); }
static size_t plan_workspace_bytes(const Plan& pl, int64_t M, int64_t R) {
    if (pl.sk) return sk_slot_bytes(pl) + sk_ticket_bytes(pl);
    return pl.splits > 1 ? (size_t)pl.splits * (size_t)M * (size_t)R * 4 : 0;
}

// group: quantization group size, or 0 when unknown (the skinny path needs 64, 128 or 256)
// allow_balanced = false asks for the plan a caller with too little workspace for the balanced one falls back to.
static Plan make_plan(int kind, int64_t M, int64_t N, int64_t K, int group = 128, bool allow_balanced = true) {
    Plan pl{};
    if (kind == KIND_FWD && M <= 16 && (K % 256) == 0 && (group == 64 || group == 128 || group == 256) && !getenv("LQ_GEMM_NO_SKINNY")) {
        // decode-sized forward: bandwidth-bound register-dequant kernel (lq_gemv.cu)
        pl.skinny = true;
        if (skinny_rows_supported(K, group) && !getenv("LQ_SKINNY_SPLIT")) { pl.splits = 1; pl.kb_per_split = (int)(K / 64); pl.kb_total = (int)(K / 64); return pl; }
        pl.kb_per_split = skinny_chunks_per_split(N, K, &pl.splits);
        pl.kb_total = (int)(K / 64);
        return pl;
    }
    const int64_t R = (kind == KIND_DGRAD) ? K : N;
    const int64_t Cc = (kind == KIND_DGRAD) ? N : K;
    pl.tn = M <= 16 ? 16 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
    pl.t_tiles = (int)((M + pl.tn - 1) / pl.tn);
    const int r_tiles1 = (int)((R + TILE_R - 1) / TILE_R);
    pl.rt = 1;   // the kernel template supports two weight-row tiles per CTA (RT = 2); no current plan uses it
    pl.r_tiles = (r_tiles1 + pl.rt - 1) / pl.rt;
    const int bk = (kind == KIND_I8) ? 128 : 64;
    pl.kb_total = (int)((Cc + bk - 1) / bk);
    const int tiles = pl.r_tiles * pl.t_tiles;
    const int sms = sm_count();
    // Balanced forward, opt-in with LQ_GEMM_BALANCE=1 (read at every launch).  With few tiles per SM, whole tiles
    // leave SMs idle or a last wave nearly empty (86 tiles of a 11008-row layer on 148 SMs; 172 tiles at 512 tokens =
    // one full wave and one of 24 tiles).  The tiles of the last, incomplete wave can be shared instead: an owner
    // computes the head of the k range, the CTAs without a tile of their own the tails (see SegWalk); the head is
    // sized so that the helpers finish `margin` k-blocks before the owners.  Measured on the four Llama-2-7B shapes
    // it does not pay: adding up a tile's parts and the epilogue behind it are ~14 k cycles of single-warp-per-lane-
    // quarter work at the very end (470 cycles per 16-column slab and part), as much as the ~13 k cycles the shorter
    // main loop saves (41 us against 25 us for the 11008-row layer at 128 tokens), so whole tiles stay the default.
    if (kind == KIND_FWD && pl.tn >= 64 && allow_balanced && (pl.tn < 256 || a_operand_in_tmem(kind))) {
        const char* e = getenv("LQ_GEMM_BALANCE");
        const bool off = !e || e[0] == '0', force = e && e[0] == '1';
        const int kb = pl.kb_total;
        const int full = tiles / sms * sms, rem = tiles - full;
        const int margin = 4 + pl.tn / 64;
        int helpers = sms - rem, h = 0;
        if (helpers > 6 * rem) helpers = 6 * rem;                   // a tile's sums are added up by one CTA: bound its parts
        bool found = false;
        for (int it = 0; it < 16 && rem > 0 && helpers > 0 && !off; ++it) {
            h = (rem * kb + margin * helpers + rem + helpers - 1) / (rem + helpers);
            if (h < 1) h = 1;
            const int tail_units = rem * (kb - h);
            if (h >= kb || tail_units < 2) break;
            if (tail_units >= 4 * helpers) { found = true; break; }
            helpers = tail_units / 4;                               // at least four k-blocks per helper
        }
        if (found && force) {
            pl.sk = true; pl.splits = 1; pl.kb_per_split = kb;
            pl.sk_full = full; pl.sk_rem = rem; pl.sk_h = h; pl.sk_helpers = helpers;
            pl.sk_grid = full > 0 ? sms : rem + helpers;
            const int share = rem * (kb - h) / helpers;             // smallest helper range
            pl.sk_pmax = 1 + (kb - h + share - 1) / share + 1;
            return pl;
        }
    }
    int splits = 1;
    if (tiles * 2 <= sms) {
        splits = sms / tiles;
        if (splits > pl.kb_total / 4) splits = pl.kb_total / 4;   // at least 4 k-blocks per item
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    pl.kb_per_split = (pl.kb_total + splits - 1) / splits;
    pl.splits = (pl.kb_total + pl.kb_per_split - 1) / pl.kb_per_split;
    return pl;
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled get_encode() {
    static PFN_encodeTiled fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(f);
    }
    return fn;
}
// 2-D row-major tensor [rows, cols] of `elt` bytes; box [box_rows, box_cols].
static int make_map(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elt, uint64_t rows, uint64_t cols,
                    uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
    PFN_encodeTiled enc = get_encode();
    if (!enc) return LQ_ECUDA;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * (uint64_t)elt};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled"); return LQ_ECUDA; }
    return LQ_OK;
}

template <int KIND, int TN, int RT, bool TA = false, bool SK = false, bool QPT = false>
static int launch_tn(const CUtensorMap& mt, const CUtensorMap& mw, const GemmParams& p, cudaStream_t st, int sk_grid = 0) {
    using C = Cfg<KIND, TN, RT, TA, SK>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm<KIND, TN, RT, TA, SK, QPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute"); return LQ_ECUDA; }
        attr_done[dev] = true;
    }
    if (SK) {
        // hand-over tickets start at zero in every launch (a memset node when the launch is being captured)
        unsigned char* tickets = reinterpret_cast<unsigned char*>(p.partial) + (size_t)p.sk_rem * p.sk_pmax * (size_t)TN * TILE_R * 4;
        cudaError_t e = cudaMemsetAsync(tickets, 0, (size_t)p.sk_rem * 4 * sizeof(unsigned int), st);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaMemsetAsync(hand-over tickets)"); return LQ_ECUDA; }
        k_gemm<KIND, TN, RT, TA, SK, QPT><<<sk_grid, C::THREADS, C::SMEM_BYTES, st>>>(mt, mw, p);
        return check_launch("k_gemm (balanced)");
    }
    const int items = p.r_tiles * p.t_tiles * p.splits;
    const int grid = items < sm_count() ? items : sm_count();
    k_gemm<KIND, TN, RT, TA, SK, QPT><<<grid, C::THREADS, C::SMEM_BYTES, st>>>(mt, mw, p);
    int rc = check_launch("k_gemm");
    if (rc) return rc;
    if (p.splits > 1) {
        const int64_t total = (int64_t)p.M * p.R;
        int g = (int)((total + 255) / 256);
        if (g > sm_count() * 8) g = sm_count() * 8;
        k_splitk_reduce<KIND == KIND_I8><<<g, 256, 0, st>>>(p);
        rc = check_launch("k_splitk_reduce");
    }
    return rc;
}
// balanced forward (token tiles of 64 / 128 / 256), either placement of the weight tile
template <bool TA>
static int launch_fwd_sk(int tn, const CUtensorMap& mt, const CUtensorMap& mw, const GemmParams& p, cudaStream_t st, int sk_grid) {
    switch (tn) {
        case 64: return launch_tn<KIND_FWD, 64, 1, TA, true>(mt, mw, p, st, sk_grid);
        case 128: return launch_tn<KIND_FWD, 128, 1, TA, true>(mt, mw, p, st, sk_grid);
        case 256:   // (with the weight tile in shared memory the staging buffers leave too few pipeline stages)
            if constexpr (TA) return launch_tn<KIND_FWD, 256, 1, TA, true>(mt, mw, p, st, sk_grid);
            break;
    }
    return LQ_EUNSUPPORTED;
}
template <int KIND>
static int launch_kind_ta(int tn, const CUtensorMap& mt, const CUtensorMap& mw, const GemmParams& p, cudaStream_t st) {
    switch (tn) {
        case 16: return launch_tn<KIND, 16, 1, true>(mt, mw, p, st);
        case 64: return launch_tn<KIND, 64, 1, true>(mt, mw, p, st);
        case 128: return launch_tn<KIND, 128, 1, true>(mt, mw, p, st);
        case 256: return launch_tn<KIND, 256, 1, true>(mt, mw, p, st);
    }
    return LQ_EUNSUPPORTED;
}
template <int KIND>
static int launch_kind(int tn, int rt, const CUtensorMap& mt, const CUtensorMap& mw, const GemmParams& p, cudaStream_t st) {
    switch (tn) {
        case 16: return launch_tn<KIND, 16, 1>(mt, mw, p, st);
        case 64: return launch_tn<KIND, 64, 1>(mt, mw, p, st);
        case 128: return launch_tn<KIND, 128, 1>(mt, mw, p, st);
        case 256: return launch_tn<KIND, 256, 1>(mt, mw, p, st);
    }
    return LQ_EUNSUPPORTED;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Grad-input through a transposed copy of the weight (see k_w4_transpose): bytes of the copy and of its packed group
// parameters, and the token count from which the two extra passes over the weight pay: they cost 18 us for a
// 4096 x 11008 weight, the GEMM saves 9 us per 1024 tokens, so the routes break even near 2048 tokens.
// LQ_GEMM_DGRAD_TRANSPOSE=0 keeps the shared-memory-A kernel, =1 takes the copy from 256 tokens.
static size_t dgrad_t_bytes(int64_t N, int64_t K) { return (size_t)N * (size_t)K / 2 + (size_t)N * (size_t)(K / 128) * 4; }
static bool dgrad_t_wanted(int64_t M, int64_t N, int64_t K, int group) {
    const char* e = getenv("LQ_GEMM_DGRAD_TRANSPOSE");
    if (e && e[0] == '0') return false;
    if (group != 128 || (K % 256) != 0 || (N % 64) != 0 || getenv("LQ_GEMM_A_OPERAND")) return false;
    return M >= ((e && e[0] == '1') ? 256 : 3072);
}
static int run_dgrad_transposed(const void* dy, const void* w, GemmParams p, int64_t M, int64_t N, int64_t K, void* workspace,
                                cudaStream_t st);

static int run_gemm(int kind, const void* tok, const void* w, GemmParams p, int64_t M, int64_t N, int64_t K,
                    void* workspace, size_t workspace_bytes, cudaStream_t st) {
    if (M == 0) return LQ_OK;
    { int rc_dev = ensure_device_for(tok); if (rc_dev) return rc_dev; }
    if (kind == KIND_DGRAD && dgrad_t_wanted(M, N, K, p.group) && workspace && workspace_bytes >= dgrad_t_bytes(N, K) &&
        (reinterpret_cast<uintptr_t>(workspace) & 15) == 0)
        return run_dgrad_transposed(tok, w, p, M, N, K, workspace, st);
    Plan pl = make_plan(kind, M, N, K, p.group);
    p.M = (int)M; p.R = (int)((kind == KIND_DGRAD) ? K : N); p.C = (int)((kind == KIND_DGRAD) ? N : K);
    // a caller whose workspace is too small for the balanced plan gets the whole-tile plan (which may need less or none)
    if (pl.sk && (!workspace || workspace_bytes < plan_workspace_bytes(pl, M, p.R))) pl = make_plan(kind, M, N, K, p.group, false);
    p.wcols = (int)K;
    p.r_tiles = pl.r_tiles; p.t_tiles = pl.t_tiles; p.splits = pl.splits; p.kb_total = pl.kb_total; p.kb_per_split = pl.kb_per_split;
    if (pl.splits > 1) {
        const size_t need = (size_t)pl.splits * (size_t)M * (size_t)p.R * 4;
        if (!workspace || workspace_bytes < need || !al16(workspace)) return LQ_EWORKSPACE;
        p.partial = workspace;
    }
    if (pl.sk) {
        if (!workspace || workspace_bytes < plan_workspace_bytes(pl, M, p.R) || !al16(workspace)) return LQ_EWORKSPACE;
        p.partial = workspace;
        p.sk_full = pl.sk_full; p.sk_rem = pl.sk_rem; p.sk_h = pl.sk_h; p.sk_helpers = pl.sk_helpers; p.sk_pmax = pl.sk_pmax;
        const int tail_units = pl.sk_rem * (pl.kb_total - pl.sk_h);
        p.sk_q = tail_units / pl.sk_helpers; p.sk_r = tail_units % pl.sk_helpers;
    }
    if (pl.skinny) {
        SkinnyParams sp{};
        sp.x = (const __nv_bfloat16*)tok; sp.qweight = (const uint8_t*)w; sp.scales = p.scales; sp.zeros = p.zeros;
        sp.bias = p.bias; sp.out = p.out; sp.partial = (float*)p.partial;
        sp.M = (int)M; sp.N = (int)N; sp.K = (int)K; sp.group = p.group; sp.splits = pl.splits; sp.chunks_per_split = pl.kb_per_split;
        if (skinny_rows_supported(K, p.group) && !getenv("LQ_SKINNY_SPLIT")) return launch_skinny_rows(sp, st);
        int rc = launch_skinny_fwd(sp, st);
        if (rc || pl.splits <= 1) return rc;
        const int64_t total = (int64_t)p.M * p.R;
        int g = (int)((total + 255) / 256);
        if (g > sm_count() * 8) g = sm_count() * 8;
        k_splitk_reduce<false><<<g, 256, 0, st>>>(p);
        return check_launch("k_splitk_reduce");
    }
    CUtensorMap mt, mw;
    int rc;
    if (kind == KIND_I8) {
        rc = make_map(&mt, tok, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)K, (uint32_t)pl.tn, 128, true);
        if (rc) return rc;
        rc = make_map(&mw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)K, TILE_R, 128, true);
    } else {
        rc = make_map(&mt, tok, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)p.C, (uint32_t)pl.tn, 64, true);
        if (rc) return rc;
        if (kind == KIND_FWD)   // packed bytes [N, K/2]; box 128 rows x 32 bytes
            rc = make_map(&mw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)(K / 2), TILE_R, 32, false);
        else                    // box 64 rows x 64 bytes
            rc = make_map(&mw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)(K / 2), 64, 64, false);
    }
    if (rc) return rc;
    switch (kind) {
        case KIND_FWD:
            if (pl.sk) return a_operand_in_tmem(kind) ? launch_fwd_sk<true>(pl.tn, mt, mw, p, st, pl.sk_grid) : launch_fwd_sk<false>(pl.tn, mt, mw, p, st, pl.sk_grid);
            return (pl.rt == 1 && a_operand_in_tmem(kind)) ? launch_kind_ta<KIND_FWD>(pl.tn, mt, mw, p, st)
                                                       : launch_kind<KIND_FWD>(pl.tn, pl.rt, mt, mw, p, st);
        case KIND_DGRAD:
            return (pl.rt == 1 && a_operand_in_tmem(kind)) ? launch_kind_ta<KIND_DGRAD>(pl.tn, mt, mw, p, st)
                                                       : launch_kind<KIND_DGRAD>(pl.tn, pl.rt, mt, mw, p, st);
        case KIND_I8: return launch_kind<KIND_I8>(pl.tn, pl.rt, mt, mw, p, st);
    }
    return LQ_EINVAL;
}

static int run_dgrad_transposed(const void* dy, const void* w, GemmParams p, int64_t M, int64_t N, int64_t K, void* workspace,
                                cudaStream_t st) {
    uint8_t* wt = reinterpret_cast<uint8_t*>(workspace);                                   // [K][N / 2]
    uint4* qpt = reinterpret_cast<uint4*>(wt + (size_t)N * (size_t)K / 2);                 // [K / 128][N / 8][2]
    const int G = (int)(K / 128);
    k_w4_transpose<<<dim3((unsigned)(K / 256), (unsigned)(N / 64)), 256, 0, st>>>(reinterpret_cast<const uint8_t*>(w), wt, (int)N, (int)K);
    int rc = check_launch("k_w4_transpose");
    if (rc) return rc;
    const int entries = G * (int)(N / 8);
    k_w4_qp_transpose<<<(entries + 255) / 256, 256, 0, st>>>(p.scales, p.zeros, qpt, (int)N, G);
    rc = check_launch("k_w4_qp_transpose");
    if (rc) return rc;
    // dx[M, K] = dy[M, N] . Wt[K, N]^T: the forward kernel with K output rows and N as the contraction
    p.M = (int)M; p.R = (int)K; p.C = (int)N; p.wcols = (int)N; p.qpt = qpt;
    p.t_tiles = (int)((M + 255) / 256); p.r_tiles = (int)((K + TILE_R - 1) / TILE_R); p.splits = 1;
    p.kb_total = (int)(N / 64); p.kb_per_split = p.kb_total;
    CUtensorMap mt, mw;
    rc = make_map(&mt, dy, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, 256, 64, true);
    if (rc) return rc;
    rc = make_map(&mw, wt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)(N / 2), TILE_R, 32, false);
    if (rc) return rc;
    return launch_tn<KIND_FWD, 256, 1, true, false, true>(mt, mw, p, st);
}

}  // namespace lq

using namespace lq;

extern "C" {

size_t lq_gemm_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K) {
    if (kind < 0 || kind > 2 || M <= 0 || N <= 0 || K <= 0) return 0;
    // the forward plan depends on the group size (decode-sized kernel or tensor-core kernel): cover both
    const int64_t R = (kind == KIND_DGRAD) ? K : N;
    size_t need = 0;
    for (int group : {64, 128, 0}) {
        for (bool balanced : {true, false}) {
            const size_t b = plan_workspace_bytes(make_plan(kind, M, N, K, group, balanced), M, R);
            if (b > need) need = b;
        }
        if (kind == KIND_DGRAD && group == 128 && dgrad_t_wanted(M, N, K, group) && dgrad_t_bytes(N, K) > need) need = dgrad_t_bytes(N, K);
    }
    return need;
}

static bool shape_ok_w4(int64_t M, int64_t N, int64_t K, int group) {
    return M >= 0 && N > 0 && K > 0 && M < (1 << 30) && N < (1 << 30) && K < (1 << 30) && group >= 32 && (group % 32) == 0 &&
           (K % group) == 0 && (K % 128) == 0 && (N % 64) == 0;
}

int lq_gemm_a16w4_fwd(const void* x, const int8_t* qweight, const void* scales, const void* zeros, const void* bias, void* y,
                      int64_t M, int64_t N, int64_t K, int group, void* workspace, size_t workspace_bytes, lq_stream_t stream) {
    if (!x || !qweight || !scales || !zeros || !y || !al16(x) || !al16(qweight) || !al16(y)) return LQ_EINVAL;
    if (!shape_ok_w4(M, N, K, group)) return LQ_EUNSUPPORTED;
    GemmParams p{};
    p.group = group; p.scales = (const __nv_bfloat16*)scales; p.zeros = (const __nv_bfloat16*)zeros;
    p.bias = (const __nv_bfloat16*)bias; p.out = (__nv_bfloat16*)y; p.alpha = 1.0f;
    return run_gemm(KIND_FWD, x, qweight, p, M, N, K, workspace, workspace_bytes, (cudaStream_t)stream);
}

int lq_gemm_a16w4_dgrad(const void* dy, const int8_t* qweight, const void* scales, const void* zeros, void* dx, int64_t M,
                        int64_t N, int64_t K, int group, void* workspace, size_t workspace_bytes, lq_stream_t stream) {
    if (!dy || !qweight || !scales || !zeros || !dx || !al16(dy) || !al16(qweight) || !al16(dx)) return LQ_EINVAL;
    if (!shape_ok_w4(M, N, K, group) || (group % 128) != 0 && (128 % group) != 0) return LQ_EUNSUPPORTED;
    GemmParams p{};
    p.group = group; p.scales = (const __nv_bfloat16*)scales; p.zeros = (const __nv_bfloat16*)zeros;
    p.out = (__nv_bfloat16*)dx; p.alpha = 1.0f;
    return run_gemm(KIND_DGRAD, dy, qweight, p, M, N, K, workspace, workspace_bytes, (cudaStream_t)stream);
}

int lq_gemm_a8w8(const int8_t* x8, const int8_t* w8, const float* row_scale, const float* col_scale, float alpha,
                 const void* bias, void* y, int32_t* acc_out, int64_t M, int64_t N, int64_t K, void* workspace,
                 size_t workspace_bytes, lq_stream_t stream) {
    if (!x8 || !w8 || !y || !al16(x8) || !al16(w8)) return LQ_EINVAL;
    if (M < 0 || N <= 0 || K <= 0 || M >= (1 << 30) || N >= (1 << 30) || K >= (1 << 30) || (K % 128) != 0) return LQ_EUNSUPPORTED;
    GemmParams p{};
    p.row_scale = row_scale; p.col_scale = col_scale; p.alpha = alpha; p.bias = (const __nv_bfloat16*)bias;
    p.out = (__nv_bfloat16*)y; p.acc_out = acc_out;
    return run_gemm(KIND_I8, x8, w8, p, M, N, K, workspace, workspace_bytes, (cudaStream_t)stream);
}

int lq_gemm_a16w4_fwd_silu(const void* x, const int8_t* qweight, const void* scales, const void* zeros, void* act, int64_t M,
                           int64_t I, int64_t K, int group, int hf_rounding, lq_stream_t stream) {
    if (!x || !qweight || !scales || !zeros || !act || !al16(x) || !al16(qweight) || !al16(act)) return LQ_EINVAL;
    if (!shape_ok_w4(M, 2 * I, K, group) || (I % 8) != 0) return LQ_EUNSUPPORTED;
    // the fused epilogue exists in the decode-sized row-block kernels only (a thread there holds gate[f] and up[f])
    if (M > 16 || (K % 256) != 0 || !skinny_rows_supported(K, group)) return LQ_EUNSUPPORTED;
    if (M == 0) return LQ_OK;
    { int rc_dev = ensure_device_for(x); if (rc_dev) return rc_dev; }
    SkinnyParams sp{};
    sp.x = (const __nv_bfloat16*)x; sp.qweight = (const uint8_t*)qweight; sp.scales = (const __nv_bfloat16*)scales;
    sp.zeros = (const __nv_bfloat16*)zeros; sp.out = (__nv_bfloat16*)act;
    sp.M = (int)M; sp.N = (int)I; sp.K = (int)K; sp.group = group; sp.splits = 1; sp.chunks_per_split = (int)(K / 64);
    sp.pair_stride = (int)I; sp.hf_rounding = hf_rounding;
    return launch_skinny_rows(sp, (cudaStream_t)stream);
}

int lq_gemm_a16w4_fwd_rmsnorm(const void* h, const void* delta, const void* gamma, float eps, int hf_rounding, void* h_out,
                              const int8_t* qweight, const void* scales, const void* zeros, void* y, int64_t M, int64_t N,
                              int64_t K, int group, int silu_pair, lq_stream_t stream) {
    if (!h || !gamma || !qweight || !scales || !zeros || !y || !al16(h) || !al16(gamma) || !al16(qweight) || !al16(y)) return LQ_EINVAL;
    if (delta && (!h_out || h_out == h || !al16(delta) || !al16(h_out))) return LQ_EINVAL;
    if (!shape_ok_w4(M, N, K, group) || (silu_pair && (N % 16) != 0)) return LQ_EUNSUPPORTED;
    if (!skinny_norm_supported(M, K, group) || (reinterpret_cast<uintptr_t>(scales) & 7) || (reinterpret_cast<uintptr_t>(zeros) & 7))
        return LQ_EUNSUPPORTED;
    { int rc_dev = ensure_device_for(h); if (rc_dev) return rc_dev; }
    SkinnyParams sp{};
    sp.qweight = (const uint8_t*)qweight; sp.scales = (const __nv_bfloat16*)scales; sp.zeros = (const __nv_bfloat16*)zeros;
    sp.out = (__nv_bfloat16*)y; sp.M = (int)M; sp.K = (int)K; sp.group = group; sp.splits = 1; sp.chunks_per_split = (int)(K / 64);
    sp.N = silu_pair ? (int)(N / 2) : (int)N; sp.pair_stride = silu_pair ? (int)(N / 2) : 0; sp.hf_rounding = hf_rounding;
    sp.norm_h = (const __nv_bfloat16*)h; sp.norm_delta = (const __nv_bfloat16*)delta; sp.norm_gamma = (const __nv_bfloat16*)gamma;
    sp.norm_h_out = (__nv_bfloat16*)h_out; sp.norm_eps = eps; sp.norm_hf = hf_rounding;
    return launch_skinny_rows(sp, (cudaStream_t)stream);
}

int lq_gemm_a16w4_fwd_qkv_rope(const void* x, const void* h, const void* delta, const void* gamma, float eps, void* h_out,
                               const int8_t* qweight, const void* scales, const void* zeros, void* qkv, const int64_t* positions,
                               const float* inv_freq, void* k_cache, void* v_cache, int64_t M, int Hq, int Hkv, int hd, int64_t K,
                               int group, int64_t max_len, int tokens_per_seq, int hf_rounding, lq_stream_t stream) {
    if (!qweight || !scales || !zeros || !qkv || !positions || !inv_freq || !k_cache || !v_cache || !al16(qweight) || !al16(qkv))
        return LQ_EINVAL;
    if (gamma ? (!h || !al16(h) || !al16(gamma) || (delta && (!h_out || h_out == h || !al16(delta) || !al16(h_out)))) : (!x || !al16(x)))
        return LQ_EINVAL;
    if (Hq < 1 || Hkv < 1 || (Hq % Hkv) != 0 || hd < 16 || hd > 512 || (hd % 16) != 0 || tokens_per_seq < 1 || max_len < 1 ||
        max_len >= (1ll << 31) || Hq + 2 * Hkv > 65535)
        return LQ_EUNSUPPORTED;
    const int64_t N = (int64_t)(Hq + 2 * Hkv) * hd;
    if (!shape_ok_w4(M, N, K, group) || M > 16 || !skinny_rows_supported(K, group) || getenv("LQ_SKINNY_SPLIT")) return LQ_EUNSUPPORTED;
    if (gamma && (!skinny_norm_supported(M, K, group) || (reinterpret_cast<uintptr_t>(scales) & 7) || (reinterpret_cast<uintptr_t>(zeros) & 7)))
        return LQ_EUNSUPPORTED;
    if (M == 0) return LQ_OK;
    { int rc_dev = ensure_device_for(qkv); if (rc_dev) return rc_dev; }
    SkinnyParams sp{};
    sp.x = (const __nv_bfloat16*)x; sp.qweight = (const uint8_t*)qweight; sp.scales = (const __nv_bfloat16*)scales;
    sp.zeros = (const __nv_bfloat16*)zeros; sp.out = (__nv_bfloat16*)qkv; sp.M = (int)M; sp.K = (int)K; sp.group = group;
    sp.splits = 1; sp.chunks_per_split = (int)(K / 64);
    sp.N = (int)(N / 2); sp.pair_stride = hd / 2; sp.hf_rounding = hf_rounding;       // N counts rotation pairs
    sp.rope_pos = (const long long*)positions; sp.rope_inv_freq = inv_freq; sp.rope_k = (__nv_bfloat16*)k_cache;
    sp.rope_v = (__nv_bfloat16*)v_cache; sp.rope_hd = hd; sp.rope_hq = Hq; sp.rope_hkv = Hkv; sp.rope_max_len = (int)max_len;
    sp.rope_tps = tokens_per_seq;
    if (gamma) {
        sp.norm_h = (const __nv_bfloat16*)h; sp.norm_delta = (const __nv_bfloat16*)delta; sp.norm_gamma = (const __nv_bfloat16*)gamma;
        sp.norm_h_out = (__nv_bfloat16*)h_out; sp.norm_eps = eps; sp.norm_hf = hf_rounding;
    }
    return launch_skinny_rows(sp, (cudaStream_t)stream);
}

int lq_gemm_wgrad(const void* dy, const void* x, void* dw, int64_t M, int64_t N, int64_t K, int accumulate, lq_stream_t stream) {
    if (!dy || !x || !dw || !al16(dy) || !al16(x) || !al16(dw)) return LQ_EINVAL;
    if (M < 0 || N <= 0 || K <= 0 || M >= (1 << 30) || N >= (1 << 30) || K >= (1 << 30) || (N % 8) != 0 || (K % 8) != 0) return LQ_EUNSUPPORTED;
    if (M == 0) {
        if (accumulate) return LQ_OK;
        cudaError_t e = cudaMemsetAsync(dw, 0, (size_t)N * (size_t)K * 2, (cudaStream_t)stream);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaMemsetAsync"); return LQ_ECUDA; }
        return LQ_OK;
    }
    { int rc_dev = ensure_device_for(dy); if (rc_dev) return rc_dev; }
    const int tn = K > 128 ? 256 : (K > 64 ? 128 : 64);
    GemmParams p{};
    p.M = (int)K; p.R = (int)N; p.C = (int)M; p.wcols = (int)K; p.group = 0;
    p.r_tiles = (int)((N + TILE_R - 1) / TILE_R); p.t_tiles = (int)((K + tn - 1) / tn); p.splits = 1;
    p.kb_total = (int)((M + 63) / 64); p.kb_per_split = p.kb_total;
    p.out = (__nv_bfloat16*)dw; p.alpha = 1.0f; p.accumulate = accumulate ? 1 : 0;
    CUtensorMap mt, mw;
    // both operands are read as [64 tokens] x [64 features] boxes (128-byte rows, 128B swizzle): MN-major MMA atoms
    int rc = make_map(&mt, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, 64, 64, true);
    if (rc) return rc;
    rc = make_map(&mw, dy, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, 64, 64, true);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (tn) {
        case 64: return launch_tn<KIND_WGRAD, 64, 1>(mt, mw, p, st);
        case 128: return launch_tn<KIND_WGRAD, 128, 1>(mt, mw, p, st);
        default: return launch_tn<KIND_WGRAD, 256, 1>(mt, mw, p, st);
    }
}

int lq_gemm_profile(int enable, unsigned long long* out16) {
    unsigned long long z[16] = {};
    cudaError_t e = cudaSuccess;
    if (out16) e = cudaMemcpyFromSymbol(out16, g_gemm_prof, sizeof(z));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_gemm_prof, z, sizeof(z));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_gemm_prof_on, &enable, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e, "lq_gemm_profile"); return LQ_ECUDA; }
    return LQ_OK;
}

int lq_gemm_device_status(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e, "lq_gemm_device_status"); return LQ_ECUDA; }
    if (reset && v) { int z = 0; cudaMemcpyToSymbol(g_gemm_status, &z, sizeof(int)); }
    return v ? LQ_ETIMEOUT : LQ_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Forward GEMM with built-in scratch (no caller workspace, no allocation of any kind)
// ---------------------------------------------------------------------------------------------
// Split-K partial sums of the decode-sized forward GEMM normally live in a workspace the caller
// allocates.  Some callers cannot allocate at all: code running inside a framework that owns every
// byte of device memory through its own pool, serving loops that must not hit the implicit
// device-wide synchronisation of cudaMalloc/cudaFree, and plugin hosts that forbid driver
// allocations once initialisation is over.  For them the partial sums go into this fixed array.
// It is part of the library image: every GPU that loads liblatentq holds these bytes until the
// process exits, whether or not the entry point is ever called.
#define LQ_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_fwd_static_scratch[LQ_STATIC_SCRATCH_BYTES];

// The array's name is only a host-side handle; the device address has to be asked for, once per
// device, with that device current.
static int fwd_static_scratch_ptr(void** out) {
    static void* cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { lq::set_cuda_error(e, "cudaGetDevice"); return LQ_ECUDA; }
    if (dev < 0 || dev >= 64) return LQ_EUNSUPPORTED;
    if (!cached[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_fwd_static_scratch);
        if (e != cudaSuccess || !ptr) { lq::set_cuda_error(e, "cudaGetSymbolAddress(g_fwd_static_scratch)"); return LQ_ECUDA; }
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return LQ_OK;
}

extern "C" {

size_t lq_gemm_a16w4_fwd_static_max_bytes(void) { return (size_t)LQ_STATIC_SCRATCH_BYTES; }

int lq_gemm_a16w4_fwd_static(const void* x, const int8_t* qweight, const void* scales, const void* zeros, const void* bias,
                             void* y, int64_t M, int64_t N, int64_t K, int group, lq_stream_t stream) {
    if (!x || !qweight || !scales || !zeros || !y || !al16(x) || !al16(qweight) || !al16(y)) return LQ_EINVAL;
    if (!shape_ok_w4(M, N, K, group)) return LQ_EUNSUPPORTED;
    // Partial sums needed by this shape's split-K plan; shapes that need more than the array holds are refused
    // (host arithmetic only, before anything touches the device).
    // (the balanced plan is used when its slots fit the array, else the whole-tile plan, as with any too-small workspace)
    Plan pl = make_plan(KIND_FWD, M, N, K, group);
    if (pl.sk && plan_workspace_bytes(pl, M, N) > (size_t)LQ_STATIC_SCRATCH_BYTES) pl = make_plan(KIND_FWD, M, N, K, group, false);
    const size_t need = plan_workspace_bytes(pl, M, N);
    if (need > (size_t)LQ_STATIC_SCRATCH_BYTES) {
        lq::set_cuda_error(cudaErrorInvalidValue, "lq_gemm_a16w4_fwd_static: shape needs more scratch than the built-in 8 MiB; "
                                                  "use lq_gemm_a16w4_fwd with a workspace");
        return LQ_EWORKSPACE;
    }
    // Bind the device that owns the operands BEFORE asking for the array's address: on a host thread without a
    // current context the symbol query would otherwise bind device 0 and hand back device 0's copy of the array.
    { int rc_dev = ensure_device_for(x); if (rc_dev) return rc_dev; }
    void* scratch = nullptr;
    int rc = fwd_static_scratch_ptr(&scratch);
    if (rc) return rc;
    GemmParams p{};
    p.group = group; p.scales = (const __nv_bfloat16*)scales; p.zeros = (const __nv_bfloat16*)zeros;
    p.bias = (const __nv_bfloat16*)bias; p.out = (__nv_bfloat16*)y; p.alpha = 1.0f;
    // Every partial-sum element the reduction reads is written by this launch first, so nothing in the
    // array has to start at zero and the previous call's leftovers are harmless.
    return run_gemm(KIND_FWD, x, qweight, p, M, N, K, scratch, (size_t)LQ_STATIC_SCRATCH_BYTES, (cudaStream_t)stream);
}

int lq_gemm_a16w4_fwd_static_peek(float* host_out, size_t first_float, size_t n_floats) {
    if (!host_out || (first_float + n_floats) * 4 > (size_t)LQ_STATIC_SCRATCH_BYTES) return LQ_EINVAL;
    cudaError_t e = cudaMemcpyFromSymbol(host_out, g_fwd_static_scratch, n_floats * 4, first_float * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { lq::set_cuda_error(e, "cudaMemcpyFromSymbol(g_fwd_static_scratch)"); return LQ_ECUDA; }
    return LQ_OK;
}

}  // extern "C"
