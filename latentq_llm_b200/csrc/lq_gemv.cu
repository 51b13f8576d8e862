// Decode-sized A16W4 forward (M <= 16 tokens): bandwidth-bound split-K kernel.
//   y[M,N] = x[M,K] · deq(Wq)[N,K]^T   (QLinearFunctionW4_eval.forward, utils/quant.py:149-158, as generate.py uses it)
//
// The packed int4 weights are read exactly once, 8 bytes per thread per row straight from global memory into
// registers and fed as the A operand of mma.sync.m16n8k16 (16 weight rows x 16 k) as the exact bf16 integers
// 128 + q; scale and zero point are applied once per (row, group) to the fp32 group sums:
//     sum_k x_k (q_k - z) s  =  s * ( sum_k x_k (128 + q_k)  -  (128 + z) * sum_k x_k ),
// which costs one logic op per two weights in the inner loop instead of a subtract and a multiply per weight
// (and does not round the dequantised weight to bf16, so it is slightly closer to exact arithmetic than the
// reference's bf16 weight matrix; outputs are compared with the 1e-2 relative tolerance).  The tokens are the
// 8-wide B operand, staged once per CTA in shared memory in the k-order the register extraction produces (a
// contraction does not care about the order of k as long as both operands agree), so no byte shuffles are
// needed.  Split-K partial sums go to the caller's workspace and are reduced by the GEMM's deterministic
// reduction kernel.
// Tensor-core rate is irrelevant here (the kernel is HBM-bound); tcgen05 serves the large-M path.
#include "lq_common.cuh"
#include "lq_gemv.h"

namespace lq {

__device__ __forceinline__ uint32_t sk_bf2(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 sk_u2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// silu(gate) * up on bf16 projection outputs, as the standalone kernel computes it
__device__ __forceinline__ float silu_mul_bf16(float gate, float up, int hf_rounding) {
    float s = gate / (1.0f + expf(-gate));
    if (hf_rounding) s = bf16r(s);
    return __fmul_rn(s, up);
}

// Rotary embedding + cache write for one (token, rotation pair) of a q|k|v projection block (see SkinnyParams):
// x / yv are the bf16-rounded projections of elements i and i + hd/2 of the head that pair block `blk` belongs to.
__device__ __forceinline__ void rope_store(const SkinnyParams& p, int blk, int fi, int tok, float x, float yv) {
    const int hd = p.rope_hd, half = hd >> 1, bph = hd >> 4;
    const int head = blk / bph, i = (blk - head * bph) * 8 + fi;
    const long long pos = p.rope_pos[tok];
    const bool pos_ok = pos >= 0 && pos < p.rope_max_len;
    const int b = tok / p.rope_tps;
    __nv_bfloat16* dst = p.out + (size_t)tok * (size_t)(2 * p.N) + (size_t)head * hd;
    const __nv_bfloat16 rx = __float2bfloat16_rn(x), ry = __float2bfloat16_rn(yv);
    if (head >= p.rope_hq + p.rope_hkv) {                     // v: as projected, into the buffer and the cache
        dst[i] = rx; dst[i + half] = ry;
        if (pos_ok) {
            __nv_bfloat16* c = p.rope_v + (((size_t)b * p.rope_hkv + (head - p.rope_hq - p.rope_hkv)) * p.rope_max_len + (size_t)pos) * hd;
            c[i] = rx; c[i + half] = ry;
        }
        return;
    }
    float sn, cs;
    sincosf((float)pos * p.rope_inv_freq[i], &sn, &cs);
    float ox, oy;
    if (p.hf_rounding) {      // cos / sin cast to bf16, then q*cos + rotate_half(q)*sin as bf16 tensor ops
        cs = bf16r(cs); sn = bf16r(sn);
        ox = __fadd_rn(bf16r(__fmul_rn(x, cs)), bf16r(__fmul_rn(-yv, sn)));
        oy = __fadd_rn(bf16r(__fmul_rn(yv, cs)), bf16r(__fmul_rn(x, sn)));
    } else {
        ox = __fsub_rn(__fmul_rn(x, cs), __fmul_rn(yv, sn));
        oy = __fadd_rn(__fmul_rn(x, sn), __fmul_rn(yv, cs));
    }
    const __nv_bfloat16 bx = __float2bfloat16_rn(ox), by = __float2bfloat16_rn(oy);
    if (head < p.rope_hq) { dst[i] = bx; dst[i + half] = by; return; }               // q: rotated in the buffer
    dst[i] = rx; dst[i + half] = ry;                                                  // k: as projected in the buffer
    if (pos_ok) {
        __nv_bfloat16* c = p.rope_k + (((size_t)b * p.rope_hkv + (head - p.rope_hq)) * p.rope_max_len + (size_t)pos) * hd;
        c[i] = bx; c[i + half] = by;
    }
}

// 8 codes of one packed word -> 4 bf16 pairs (128 + c_k, 128 + c_{k+4}) for k = 0..3: a nibble pair is OR-ed into the
// mantissas of two bf16 128.0 by ONE three-input logic instruction.  Written as inline PTX on scalars: the same
// expression on arrays (`((w >> 4) & MASK) | MAGIC` into p[0..3], fragments gathered into a0[4] / a1[4]) compiled to
// 9.6 integer-pipe instructions per word instead of 7 (ncu counters), and that pipe bounds these kernels.
__device__ __forceinline__ uint32_t lop_nib(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(r) : "r"(w));
    return r;
}
// A fragments of the two k-steps (16 k each) that one packed word of row a (va) and of row b (vb) covers:
// {a00, a01, a02, a03} = (row a: c0 c4 | row b: c0 c4 | row a: c1 c5 | row b: c1 c5), {a10..a13} the same for c2 c6 | c3 c7
#define LQ_WORD_FRAGS(va, vb)                                                                                          \
    const uint32_t a00 = lop_nib((va) >> 4), a01 = lop_nib((vb) >> 4), a02 = lop_nib(va), a03 = lop_nib(vb);            \
    const uint32_t a10 = lop_nib((va) >> 12), a11 = lop_nib((vb) >> 12), a12 = lop_nib((va) >> 8), a13 = lop_nib((vb) >> 8)
__device__ __forceinline__ void mma_s(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = a * b (no accumulator input: starts a new group sum without clearing registers first)
__device__ __forceinline__ void mma_s_start(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

constexpr int SK_THREADS = 256;       // 8 warps x 16 weight rows = 128 rows per CTA
constexpr int SK_ROWS = 128;
constexpr int SK_CHUNK = 64;          // k per loop step: 4 mma k-steps
constexpr int SK_XPAD = 8;            // bf16 elements of padding per token row (bank-conflict relief)

// MT = number of 8-token groups (1: M <= 8, 2: M <= 16)
template <int MT>
__global__ void __launch_bounds__(SK_THREADS) k_skinny_fwd(const SkinnyParams p) {
    extern __shared__ __align__(16) uint8_t sk_smem[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(sk_smem);
    const int chunks = p.chunks_per_split;
    const int split = blockIdx.y;
    const int c_begin = split * chunks, c_end = min(p.K / SK_CHUNK, c_begin + chunks);
    const int n_chunks = c_end - c_begin;
    const int xstride = chunks * SK_CHUNK + SK_XPAD;            // elements per token row in smem

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * SK_ROWS + warp * 16;
    const int ra = min(row0 + g, p.N - 1), rb = min(row0 + g + 8, p.N - 1);        // clamped loads, guarded stores
    const size_t row_bytes = (size_t)p.K / 2;
    const uint8_t* wa = p.qweight + (size_t)ra * row_bytes + (size_t)c_begin * (SK_CHUNK / 2) + t * 8;
    const uint8_t* wb = p.qweight + (size_t)rb * row_bytes + (size_t)c_begin * (SK_CHUNK / 2) + t * 8;
    const int gpr = p.K / p.group;
    const unsigned short* sca = reinterpret_cast<const unsigned short*>(p.scales) + (size_t)ra * gpr;
    const unsigned short* scb = reinterpret_cast<const unsigned short*>(p.scales) + (size_t)rb * gpr;
    const unsigned short* zpa = reinterpret_cast<const unsigned short*>(p.zeros) + (size_t)ra * gpr;
    const unsigned short* zpb = reinterpret_cast<const unsigned short*>(p.zeros) + (size_t)rb * gpr;

    // packed weights of one chunk (2 rows x 16 k per thread); PF chunks are in flight per thread, issued before the
    // token tile is staged so that the weight stream starts with the kernel
    struct Chunk { uint2 qa, qb; };
    auto load_chunk = [&](int c) -> Chunk {
        Chunk ck;
        ck.qa = __ldg(reinterpret_cast<const uint2*>(wa + (size_t)c * (SK_CHUNK / 2)));
        ck.qb = __ldg(reinterpret_cast<const uint2*>(wb + (size_t)c * (SK_CHUNK / 2)));
        return ck;
    };
    constexpr int PF = 4;
    Chunk ring[PF];
#pragma unroll
    for (int u = 0; u < PF; ++u) {
        ring[u].qa = ring[u].qb = make_uint2(0, 0);
        if (u < n_chunks) ring[u] = load_chunk(u);
    }
    const int gc = p.group / SK_CHUNK;                      // chunks per quantization group (slices hold whole groups)
    const int g_first = c_begin / gc, n_groups = (n_chunks + gc - 1) / gc;
    // (scale, zero) of the first group for both rows, prefetched one group ahead inside the loop
    uint32_t sz_a = (uint32_t)__ldg(sca + g_first) | ((uint32_t)__ldg(zpa + g_first) << 16);
    uint32_t sz_b = (uint32_t)__ldg(scb + g_first) | ((uint32_t)__ldg(zpb + g_first) << 16);

    // stage x[0..8*MT) x [k slice] with every 8-run of k reordered to (0,4,1,5,2,6,3,7)
    for (int i = threadIdx.x; i < MT * 8 * n_chunks * (SK_CHUNK / 8); i += SK_THREADS) {
        const int run = i % (n_chunks * (SK_CHUNK / 8));
        const int tok = i / (n_chunks * (SK_CHUNK / 8));
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < p.M) v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)tok * p.K + (size_t)c_begin * SK_CHUNK) + run);
        uint4 o;   // (k0,k1)(k2,k3)(k4,k5)(k6,k7) -> (k0,k4)(k1,k5)(k2,k6)(k3,k7)
        o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
        *reinterpret_cast<uint4*>(xs + (size_t)tok * xstride + run * 8) = o;
    }
    __syncthreads();
    const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};   // bf16 1.0
    float tot[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) { tot[m][0] = tot[m][1] = tot[m][2] = tot[m][3] = 0.0f; }

    int c = 0;
    for (int grp = 0; grp < n_groups; ++grp) {
        const uint32_t cur_a = sz_a, cur_b = sz_b;
        if (grp + 1 < n_groups) {
            sz_a = (uint32_t)__ldg(sca + g_first + grp + 1) | ((uint32_t)__ldg(zpa + g_first + grp + 1) << 16);
            sz_b = (uint32_t)__ldg(scb + g_first + grp + 1) | ((uint32_t)__ldg(zpb + g_first + grp + 1) << 16);
        }
        float acc[MT][4], sx[MT][4];      // sx: sum of the activations over the group, from an all-ones A operand
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;
            sx[m][0] = sx[m][1] = sx[m][2] = sx[m][3] = 0.0f;
        }
        const int c_stop = min(n_chunks, (grp + 1) * gc);
        for (; c < c_stop; ++c) {
            const int u = c % PF;
            Chunk ck;
            // the ring is indexed with a runtime slot; PF is small, so select with predicates instead of local memory
            ck = ring[0];
#pragma unroll
            for (int q = 1; q < PF; ++q) if (u == q) ck = ring[q];
            if (c + PF < n_chunks) {
                const Chunk nx = load_chunk(c + PF);
#pragma unroll
                for (int q = 0; q < PF; ++q) if (u == q) ring[q] = nx;
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {          // the chunk's two packed words per row: 2 x 2 k-steps
                LQ_WORD_FRAGS(half ? ck.qa.y : ck.qa.x, half ? ck.qb.y : ck.qb.x);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const __nv_bfloat16* xr = xs + (size_t)(m * 8 + g) * xstride + c * SK_CHUNK + t * 16 + half * 8;
                    const uint4 xv = *reinterpret_cast<const uint4*>(xr);
                    mma_s(acc[m], a00, a01, a02, a03, xv.x, xv.y);
                    mma_16816(sx[m], ones, xv.x, xv.y);
                    mma_s(acc[m], a10, a11, a12, a13, xv.z, xv.w);
                    mma_16816(sx[m], ones, xv.z, xv.w);
                }
            }
        }
        // fold the group: s * (sum x (128 + q) - (128 + z) * sum x)
        const float s_a = __uint_as_float(cur_a << 16), z_a = __uint_as_float(cur_a & 0xffff0000u) + 128.0f;
        const float s_b = __uint_as_float(cur_b << 16), z_b = __uint_as_float(cur_b & 0xffff0000u) + 128.0f;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float sx0 = sx[m][0], sx1 = sx[m][1];      // tokens 2t, 2t+1 (identical in every row of the ones tile)
            tot[m][0] = fmaf(s_a, acc[m][0] - z_a * sx0, tot[m][0]);
            tot[m][1] = fmaf(s_a, acc[m][1] - z_a * sx1, tot[m][1]);
            tot[m][2] = fmaf(s_b, acc[m][2] - z_b * sx0, tot[m][2]);
            tot[m][3] = fmaf(s_b, acc[m][3] - z_b * sx1, tot[m][3]);
        }
    }
    float (&acc)[MT][4] = tot;

    // D fragment: d0,d1 = (row g, tokens 2t, 2t+1); d2,d3 = (row g+8, same tokens)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + g + ((i >= 2) ? 8 : 0);
            const int tok = m * 8 + 2 * t + (i & 1);
            if (row >= p.N || tok >= p.M) continue;
            const size_t o = (size_t)tok * p.N + row;
            if (p.splits > 1) {
                p.partial[(size_t)split * p.M * p.N + o] = acc[m][i];
            } else {
                const float f = bf16r(acc[m][i]);
                p.out[o] = __float2bfloat16_rn(p.bias ? __fadd_rn(f, __bfloat162float(p.bias[row])) : f);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Row-block variant (group size 128 or 256): one CTA owns 16 weight rows over the whole K; its 8 warps split K
// (whole quantization groups each) and their partial sums meet in shared memory in a fixed order.  No partial sums
// in global memory, no second kernel: one launch per layer, which is what a decode step is made of.  A thread
// reads 16 bytes (32 weights) of each of its two rows per 128-k chunk, so a row is fetched as 64 contiguous bytes
// per warp instruction.  Tokens are read straight from global memory (a few KB, L1/L2 resident) and reordered in
// registers to the k-order of the nibble extraction.  The loop body is straight-line code per chunk: the kernel is
// bound by instruction issue as much as by HBM, every instruction per byte counts.
// ---------------------------------------------------------------------------------------------
constexpr int RB_WARPS = 8;
constexpr int RB_CHUNK = 128;         // k per chunk

// GC = chunks per quantization group (1: group 128, 2: group 256).  MT = 1 (up to 8 tokens) keeps 4 weight chunks
// (2 rows x 16 bytes each) in flight per thread and prefetches the token fragment one chunk ahead; MT = 2 has twice
// the token registers and runs with 2 chunks and no token prefetch instead of spilling (measured faster each way).
// NC4: K = 4096 with groups of 128, i.e. exactly four chunks per warp.  The chunk loop is then written out (constant
// trip count: every token and weight offset is a compile-time constant) and a row's four (scale, zero) pairs come as
// two 8-byte loads.
// NCH = 11: K = 11008 (86 groups: eleven chunks per warp, nine in the last warp): the same loop written out for up
// to eleven chunks, each guarded by the warp's own count; group parameters stay 2-byte loads (rows of 86 groups are
// not 8-byte aligned) but at constant offsets.
template <int MT, int GC, int NCH = 0>
__global__ void __launch_bounds__(RB_WARPS * 32, 2) k_skinny_rows(const SkinnyParams p) {
    constexpr int RB_PF = MT == 1 ? 4 : 2;
    constexpr bool XPF = MT == 1;
    constexpr bool NC4 = NCH == 4;
    static_assert(NCH == 0 || GC == 1, "the written-out loops are for group 128");
    __shared__ float red[RB_WARPS][MT][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bool pair = p.pair_stride > 0;
    const int row0 = blockIdx.x * (pair ? 8 : 16);
    const int rope_bph = p.rope_hd >> 4;                                            // pair blocks per head (rope mode)
    const int ra = p.rope_hd ? ((int)blockIdx.x / rope_bph) * p.rope_hd + ((int)blockIdx.x % rope_bph) * 8 + g
                             : min(row0 + g, p.N - 1);                              // clamped loads, guarded stores
    const int rb = pair ? p.pair_stride + ra : min(row0 + g + 8, p.N - 1);
    const int gpr = NC4 ? 32 : p.K / (RB_CHUNK * GC);                               // groups per weight row
    const int gper = NC4 ? 4 : (gpr + RB_WARPS - 1) / RB_WARPS;
    const int g_begin = NC4 ? warp * 4 : min(gpr, warp * gper), n_groups = NC4 ? 4 : min(gpr, g_begin + gper) - g_begin;
    const int n_chunks = n_groups * GC;
    const int row_bytes = NC4 ? 2048 : p.K / 2, row_elems = NC4 ? 4096 : p.K;
    const uint4* wa = reinterpret_cast<const uint4*>(p.qweight + (size_t)ra * row_bytes + (size_t)g_begin * GC * (RB_CHUNK / 2)) + t;
    const uint4* wb = reinterpret_cast<const uint4*>(p.qweight + (size_t)rb * row_bytes + (size_t)g_begin * GC * (RB_CHUNK / 2)) + t;
    const unsigned short* sca = reinterpret_cast<const unsigned short*>(p.scales) + (size_t)ra * gpr + g_begin;
    const unsigned short* scb = reinterpret_cast<const unsigned short*>(p.scales) + (size_t)rb * gpr + g_begin;
    const unsigned short* zpa = reinterpret_cast<const unsigned short*>(p.zeros) + (size_t)ra * gpr + g_begin;
    const unsigned short* zpb = reinterpret_cast<const unsigned short*>(p.zeros) + (size_t)rb * gpr + g_begin;
    // this thread's 32 k of token m*8+g inside chunk 0 of the slice (4 x 16 bytes), null when the token does not exist
    const uint4* xp[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m)
        xp[m] = (m * 8 + g < p.M) ? reinterpret_cast<const uint4*>(p.x + (size_t)(m * 8 + g) * row_elems + (size_t)g_begin * GC * RB_CHUNK + t * 32)
                                  : nullptr;

    uint4 qa[RB_PF], qb[RB_PF];
#pragma unroll
    for (int u = 0; u < RB_PF; ++u) {
        qa[u] = qb[u] = make_uint4(0, 0, 0, 0);
        if (u < n_chunks) { qa[u] = __ldg(wa + u * 4); qb[u] = __ldg(wb + u * 4); }       // a chunk is 64 bytes = 4 uint4 per row
    }
    // (scale | zero << 16) of the group that starts with the chunk in ring slot u: fetched as far ahead as the chunk
    // itself (they come from DRAM too; one group ahead was a stall per group)
    uint32_t sza[RB_PF], szb[RB_PF], sz_a = 0, sz_b = 0;
#pragma unroll
    for (int u = 0; u < RB_PF; ++u) {
        sza[u] = szb[u] = 0;
        if (!NC4 && u % GC == 0 && u < n_chunks) {
            sza[u] = (uint32_t)__ldg(sca + u / GC) | ((uint32_t)__ldg(zpa + u / GC) << 16);
            szb[u] = (uint32_t)__ldg(scb + u / GC) | ((uint32_t)__ldg(zpb + u / GC) << 16);
        }
    }
    uint2 s4a = make_uint2(0, 0), z4a = s4a, s4b = s4a, z4b = s4a;
    if (NC4) {
        s4a = __ldg(reinterpret_cast<const uint2*>(sca)); z4a = __ldg(reinterpret_cast<const uint2*>(zpa));
        s4b = __ldg(reinterpret_cast<const uint2*>(scb)); z4b = __ldg(reinterpret_cast<const uint2*>(zpb));
    }
    pdl_launch_dependents();        // weight and group-parameter loads are issued: the next launch may start
    pdl_wait();                     // the tokens may be the previous launch's output
    uint4 xn[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) xn[m][j] = (XPF && xp[m] && n_chunks > 0) ? xp[m][j] : make_uint4(0, 0, 0, 0);

    float tot[MT][4], acc[MT][2][4];     // two accumulator chains per token group
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) { tot[m][i] = acc[m][0][i] = acc[m][1][i] = 0.0f; }

    // The zero point is subtracted from the codes before the MMA (exact: small integers in bf16; zero points are
    // integer-valued) instead of being applied to token sums from an all-ones MMA: that trades half of the mma.sync
    // of a chunk (the legacy tensor path runs 0.5 per cycle per SM) for 32 half-rate packed subtractions.  Measured
    // -11 % at 16 tokens, -2 % at 4..8, and the group sum loses no bits to the cancellation of 128 * sum(x).
    __nv_bfloat162 zp2a = __float2bfloat162_rn(0.0f), zp2b = zp2a;
    auto sz_of_chunk = [&](const int c, const int u) {
        if (NC4) {          // group c of the slice: bf16 half (c & 1) of word (c >> 1) of the packed loads
            const uint32_t sw_a = c < 2 ? s4a.x : s4a.y, zw_a = c < 2 ? z4a.x : z4a.y;
            const uint32_t sw_b = c < 2 ? s4b.x : s4b.y, zw_b = c < 2 ? z4b.x : z4b.y;
            sz_a = ((c & 1) ? (sw_a >> 16) : (sw_a & 0xffffu)) | ((c & 1) ? (zw_a & 0xffff0000u) : (zw_a << 16));
            sz_b = ((c & 1) ? (sw_b >> 16) : (sw_b & 0xffffu)) | ((c & 1) ? (zw_b & 0xffff0000u) : (zw_b << 16));
        } else {
            sz_a = sza[u]; sz_b = szb[u];
        }
        const __nv_bfloat162 c128 = __float2bfloat162_rn(128.0f);          // (128 + z) in both halves
        zp2a = __hadd2_rn(sk_u2((sz_a & 0xffff0000u) | (sz_a >> 16)), c128);
        zp2b = __hadd2_rn(sk_u2((sz_b & 0xffff0000u) | (sz_b >> 16)), c128);
    };
    // chunk c of the slice, held in ring slot u (u a compile-time constant at every call)
    auto do_chunk = [&](const int c, const int u) {
        const uint4 ca = qa[u], cq = qb[u];
        if (u % GC == 0) sz_of_chunk(c, u);
        if (c + RB_PF < n_chunks) {
            qa[u] = __ldg(wa + (c + RB_PF) * 4); qb[u] = __ldg(wb + (c + RB_PF) * 4);
            if (!NC4 && u % GC == 0) {
                const int gn = (c + RB_PF) / GC;
                sza[u] = (uint32_t)__ldg(sca + gn) | ((uint32_t)__ldg(zpa + gn) << 16);
                szb[u] = (uint32_t)__ldg(scb + gn) | ((uint32_t)__ldg(zpb + gn) << 16);
            }
        }
        uint4 xc[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (XPF) {
                    xc[m][j] = xn[m][j];
                    if (xp[m] && c + 1 < n_chunks) xn[m][j] = xp[m][(c + 1) * (RB_CHUNK * 2 / 16) + j];
                } else {
                    xc[m][j] = xp[m] ? xp[m][c * (RB_CHUNK * 2 / 16) + j] : make_uint4(0, 0, 0, 0);
                }
            }
        const uint32_t wsa[4] = {ca.x, ca.y, ca.z, ca.w}, wsb[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {      // one packed word = 8 k of each row = two MMA k-steps
            LQ_WORD_FRAGS(wsa[w], wsb[w]);
            // minus (128 + z): exact in bf16, so the MMAs sum x (q - z) and no token sums are needed
            const uint32_t d00 = sk_bf2(__hsub2_rn(sk_u2(a00), zp2a)), d01 = sk_bf2(__hsub2_rn(sk_u2(a01), zp2b));
            const uint32_t d02 = sk_bf2(__hsub2_rn(sk_u2(a02), zp2a)), d03 = sk_bf2(__hsub2_rn(sk_u2(a03), zp2b));
            const uint32_t d10 = sk_bf2(__hsub2_rn(sk_u2(a10), zp2a)), d11 = sk_bf2(__hsub2_rn(sk_u2(a11), zp2b));
            const uint32_t d12 = sk_bf2(__hsub2_rn(sk_u2(a12), zp2a)), d13 = sk_bf2(__hsub2_rn(sk_u2(a13), zp2b));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint4 v = xc[m][w];  // (k0,k1)(k2,k3)(k4,k5)(k6,k7) -> (k0,k4)(k1,k5)(k2,k6)(k3,k7)
                const uint32_t x0 = __byte_perm(v.x, v.z, 0x5410), x1 = __byte_perm(v.x, v.z, 0x7632);
                const uint32_t x2 = __byte_perm(v.y, v.w, 0x5410), x3 = __byte_perm(v.y, v.w, 0x7632);
                mma_s(acc[m][0], d00, d01, d02, d03, x0, x1);
                mma_s(acc[m][1], d10, d11, d12, d13, x2, x3);
            }
        }
        if ((u + 1) % GC == 0) {
            // fold the group: tot += s * sum x (q - z)
            const float s_a = __uint_as_float(sz_a << 16), s_b = __uint_as_float(sz_b << 16);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                tot[m][0] = fmaf(s_a, acc[m][0][0] + acc[m][1][0], tot[m][0]);
                tot[m][1] = fmaf(s_a, acc[m][0][1] + acc[m][1][1], tot[m][1]);
                tot[m][2] = fmaf(s_b, acc[m][0][2] + acc[m][1][2], tot[m][2]);
                tot[m][3] = fmaf(s_b, acc[m][0][3] + acc[m][1][3], tot[m][3]);
#pragma unroll
                for (int i = 0; i < 4; ++i) { acc[m][0][i] = acc[m][1][i] = 0.0f; }
            }
        }
    };
    if constexpr (NC4) {
#pragma unroll
        for (int c = 0; c < 4; ++c) do_chunk(c, c % RB_PF);
    } else if constexpr (NCH > 0) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
            if (c < n_chunks) do_chunk(c, c % RB_PF);
    } else {
        for (int cb = 0; cb < n_chunks; cb += RB_PF) {
#pragma unroll
            for (int u = 0; u < RB_PF; ++u)          // ring slot = unroll index: no runtime register indexing
                if (cb + u < n_chunks) do_chunk(cb + u, u);
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
        *reinterpret_cast<float4*>(&red[warp][m][lane * 4]) = make_float4(tot[m][0], tot[m][1], tot[m][2], tot[m][3]);
    __syncthreads();
    // D fragment: d0,d1 = (row g, tokens 2t, 2t+1); d2,d3 = (row g+8, same tokens)
    for (int j = threadIdx.x; j < MT * 128; j += RB_WARPS * 32) {
        const int m = j >> 7, idx = j & 127, ln = idx >> 2, i = idx & 3;
        const int tok = m * 8 + 2 * (ln & 3) + (i & 1);
        if (pair) {                                            // d0,d1 = gate[f], d2,d3 = up[f] of the same tokens
            const int f = row0 + (ln >> 2);
            if (i >= 2 || f >= p.N || tok >= p.M) continue;
            float ag = 0.0f, au = 0.0f;
#pragma unroll
            for (int w = 0; w < RB_WARPS; ++w) { ag = __fadd_rn(ag, red[w][m][idx]); au = __fadd_rn(au, red[w][m][idx + 2]); }
            if (p.rope_hd) { rope_store(p, (int)blockIdx.x, ln >> 2, tok, bf16r(ag), bf16r(au)); continue; }
            p.out[(size_t)tok * p.N + f] = __float2bfloat16_rn(silu_mul_bf16(bf16r(ag), bf16r(au), p.hf_rounding));
            continue;
        }
        const int row = row0 + (ln >> 2) + ((i >= 2) ? 8 : 0);
        if (row >= p.N || tok >= p.M) continue;
        float a = 0.0f;
#pragma unroll
        for (int w = 0; w < RB_WARPS; ++w) a = __fadd_rn(a, red[w][m][idx]);
        const float f = bf16r(a);
        p.out[(size_t)tok * p.N + row] = __float2bfloat16_rn(p.bias ? __fadd_rn(f, __bfloat162float(p.bias[row])) : f);
    }
}

// ---------------------------------------------------------------------------------------------
// Streaming variant of the row-block kernel: persistent CTAs (two per SM) walk over the 16-row blocks, and a warp's
// weight loads run one row block ahead of its arithmetic, so HBM stays busy while the previous block is computed
// and reduced (the one-block-per-CTA kernel above loads, waits, computes, and only overlaps the two CTAs of an SM).
// What does not depend on the weight rows is done once per CTA instead of once per row block:
//   * the tokens are staged in shared memory already in the B-fragment order of the nibble extraction
//     ((k0,k4)(k1,k5)(k2,k6)(k3,k7) per 8 k), one 16-byte load per packed word instead of a load + four permutes
//     (M x K x 2 bytes must fit beside a second CTA; larger token blocks use k_skinny_rows);
//   * sum_k x_k per (token, group) — the zero-point term — is computed while staging and kept in shared memory,
//     instead of a second mma.sync per 16 k against an all-ones tile.
// Needs at least two quantization groups per warp (the group parameters are fetched one group ahead, across the
// row-block boundary); other shapes use k_skinny_rows.
// ---------------------------------------------------------------------------------------------
#ifndef LQ_GEMV_PF
#define LQ_GEMV_PF 4
#endif
#ifndef LQ_GEMV_MINB
#define LQ_GEMV_MINB 2
#endif
// NC4: every warp's slice is exactly four groups of 128 (K = 4096, the shape of three of a Llama-7B layer's four
// projections).  The loop is then written out for that case: a chunk's successor in the prefetch ring is always chunk
// u of the next row block, the four (scale, zero) pairs of a row come as two 8-byte loads per row block, and every
// shared-memory address is a constant offset from a per-warp base, which removes the index arithmetic that made up
// about half of the general loop's instructions.
// NCH = 11: K = 11008 (eleven chunks per warp, nine in the last): written out the same way with every chunk guarded by
// the warp's own count and 2-byte group-parameter loads at constant offsets.
// NORM: the tokens are RMSNorm(h + delta) * gamma, computed in the staging phase (see SkinnyParams).
template <int MT, int GC, int NCH, bool NORM = false>
__global__ void __launch_bounds__(RB_WARPS * 32, MT == 2 ? 1 : LQ_GEMV_MINB) k_skinny_stream(const SkinnyParams p, const int x_stride) {
    constexpr int PF = LQ_GEMV_PF;
    constexpr bool NC4 = NCH == 4;
    static_assert(NCH == 0 || (GC == 1 && PF == 4), "the written-out loops are for group 128 and a ring of four chunks");
    extern __shared__ __align__(16) uint8_t ss_smem[];
    uint4* xs = reinterpret_cast<uint4*>(ss_smem);                                               // [M][x_stride]
    float* sxs = reinterpret_cast<float*>(ss_smem + (size_t)p.M * x_stride * 16);               // [groups][8 * MT]
    __shared__ float red[2][RB_WARPS][MT][128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int gpr = p.K / (RB_CHUNK * GC);                                                      // groups per weight row

    const int gper = (gpr + RB_WARPS - 1) / RB_WARPS;
    const int g_begin = min(gpr, warp * gper), n_groups = min(gpr, g_begin + gper) - g_begin;
    const int n_chunks = n_groups * GC;
    const bool pair = p.pair_stride > 0;
    const int rows_per_blk = pair ? 8 : 16;
    const int n_blocks = (p.N + rows_per_blk - 1) / rows_per_blk;
    int blk = blockIdx.x;                                  // grid <= n_blocks
    const unsigned short* sc_all = reinterpret_cast<const unsigned short*>(p.scales);
    const unsigned short* zp_all = reinterpret_cast<const unsigned short*>(p.zeros);
    auto row_of = [&](int b, int half) {                                                           // clamped loads, guarded stores
        if (p.rope_hd) { const int bph = p.rope_hd >> 4; return (b / bph) * p.rope_hd + (b % bph) * 8 + g + half * p.pair_stride; }
        return pair ? half * p.pair_stride + min(b * 8 + g, p.N - 1) : min(b * 16 + g + half * 8, p.N - 1);
    };
    auto wptr = [&](int row) { return reinterpret_cast<const uint4*>(p.qweight + (size_t)row * (p.K / 2) + (size_t)g_begin * GC * (RB_CHUNK / 2)) + t; };
    auto load_sz = [&](int row, int grp) {
        const size_t i = (size_t)row * gpr + g_begin + grp;
        return (uint32_t)__ldg(sc_all + i) | ((uint32_t)__ldg(zp_all + i) << 16);
    };
    int ra = row_of(blk, 0), rb = row_of(blk, 1);
    const uint4 *wa = wptr(ra), *wb = wptr(rb);
    uint4 qa[PF], qb[PF];
#pragma unroll
    for (int u = 0; u < PF; ++u) {
        qa[u] = qb[u] = make_uint4(0, 0, 0, 0);
        if (u < n_chunks) { qa[u] = __ldg(wa + u * 4); qb[u] = __ldg(wb + u * 4); }
    }
    // group parameters ride in the same ring as the chunks: slot u holds those of the group its chunk starts
    uint32_t sza[PF], szb[PF], sz_a = 0, sz_b = 0;
#pragma unroll
    for (int u = 0; u < PF; ++u) {
        sza[u] = szb[u] = 0;
        if (!NC4 && u % GC == 0 && u < n_chunks) { sza[u] = load_sz(ra, u / GC); szb[u] = load_sz(rb, u / GC); }
    }
    // NC4: the row's four scales and four zero points of this warp's slice (8 bytes each; 32 groups per row, four per warp)
    auto load_s4 = [&](int row) { return __ldg(reinterpret_cast<const uint2*>(sc_all + (size_t)row * 32 + warp * 4)); };
    auto load_z4 = [&](int row) { return __ldg(reinterpret_cast<const uint2*>(zp_all + (size_t)row * 32 + warp * 4)); };
    uint2 s4a = make_uint2(0, 0), z4a = s4a, s4b = s4a, z4b = s4a;
    if (NC4) { s4a = load_s4(ra); z4a = load_z4(ra); s4b = load_s4(rb); z4b = load_z4(rb); }
    // token rows of this thread's B fragments (a token that does not exist reads the last one: its outputs are dropped)
    int xrow[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) xrow[m] = min(m * 8 + g, p.M - 1);

    // gamma is a parameter: requested before the dependency wait (NORM)
    uint4 ng[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (NORM) {
#pragma unroll
        for (int u = 0; u < 2; ++u) ng[u] = __ldg(reinterpret_cast<const uint4*>(p.norm_gamma) + tid + u * (RB_WARPS * 32));
    }
    pdl_launch_dependents();        // weight and group-parameter loads are issued: the next launch may start
    // ---- once per CTA, while the first weight loads are in flight: token fragments and per-group token sums
    for (int i = tid; i < gpr * 8 * MT; i += RB_WARPS * 32) sxs[i] = 0.0f;
    __syncthreads();
    pdl_wait();                     // the tokens may be the previous launch's output
    // one staged vector: 8 tokens' worth of k of token `tok` (word kw of its row), permuted into B-fragment order, and
    // its contribution to the token sum of its group
    // With 9-16 tokens the per-group token sums are not gathered here (26 of the 45 instructions per vector) but
    // computed after staging by each warp for its own groups: the staged fragments against an all-ones tile, 8 MMAs per
    // group and 8 tokens, whose D fragment is exactly the pair of sums the thread needs.
    constexpr bool mma_sums = MT == 2 && !NORM;
    auto stage_item = [&](const uint4& v, const int tok, const int kw, const bool on) {
        const uint32_t r[4] = {v.x, v.y, v.z, v.w};
        if constexpr (mma_sums) {
            if (on) {
                uint4 f;
                f.x = __byte_perm(v.x, v.z, 0x5410); f.y = __byte_perm(v.x, v.z, 0x7632);
                f.z = __byte_perm(v.y, v.w, 0x5410); f.w = __byte_perm(v.y, v.w, 0x7632);
                xs[(size_t)tok * x_stride + (kw & ~15) + ((kw & 3) << 2) + ((kw >> 2) & 3)] = f;
            }
            return;
        }
        float part = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) part += __uint_as_float(r[j] << 16) + __uint_as_float(r[j] & 0xffff0000u);
        if (on) {
            uint4 f;
            f.x = __byte_perm(v.x, v.z, 0x5410); f.y = __byte_perm(v.x, v.z, 0x7632);
            f.z = __byte_perm(v.y, v.w, 0x5410); f.w = __byte_perm(v.y, v.w, 0x7632);
            // word kw = chunk * 16 + t * 4 + w is stored at chunk * 16 + w * 4 + t: the four t of a word index are adjacent
            xs[(size_t)tok * x_stride + (kw & ~15) + ((kw & 3) << 2) + ((kw >> 2) & 3)] = f;
        }
#pragma unroll
        for (int o = 8 * GC; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (on && (lane & (16 * GC - 1)) == 0) sxs[(kw / (16 * GC)) * (8 * MT) + tok] = part;
    };
    if constexpr (NORM) {
        // K = 4096: 512 vectors per token, two per thread (vector tid + u * 256, as in k_add_rmsnorm_r<2>)
        float* nred = &red[0][0][0][0];
        for (int tk = 0; tk < p.M; ++tk) {
            const size_t row = (size_t)tk * 4096;
            uint4 a[2], d[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int i = tid + u * (RB_WARPS * 32);
                a[u] = __ldg(reinterpret_cast<const uint4*>(p.norm_h + row) + i);
                d[u] = p.norm_delta ? __ldg(reinterpret_cast<const uint4*>(p.norm_delta + row) + i) : make_uint4(0, 0, 0, 0);
            }
            float ss = 0.0f;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                uint32_t* w = reinterpret_cast<uint32_t*>(&a[u]);
                const uint32_t* e = reinterpret_cast<const uint32_t*>(&d[u]);
                if (p.norm_delta) {                    // residual + hidden_states: one bf16 rounding of the fp32 sum
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const __nv_bfloat162 sum = __floats2bfloat162_rn(__fadd_rn(__uint_as_float(w[j] << 16), __uint_as_float(e[j] << 16)),
                                                                         __fadd_rn(__uint_as_float(w[j] & 0xffff0000u), __uint_as_float(e[j] & 0xffff0000u)));
                        w[j] = sk_bf2(sum);
                    }
                    if (blockIdx.x == 0) reinterpret_cast<uint4*>(p.norm_h_out + row)[tid + u * (RB_WARPS * 32)] = a[u];
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
                    ss = fmaf(lo, lo, ss); ss = fmaf(hi, hi, ss);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) nred[warp] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int wv = 0; wv < RB_WARPS; ++wv) tot += nred[wv];                 // same order in every thread
            const float rstd = p.norm_hf ? rsqrtf(tot / 4096.0f + p.norm_eps) : 1.0f / sqrtf(tot / 4096.0f + p.norm_eps);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint32_t* w = reinterpret_cast<const uint32_t*>(&a[u]);
                const uint32_t* gw = reinterpret_cast<const uint32_t*>(&ng[u]);
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float lo = __fmul_rn(__uint_as_float(w[j] << 16), rstd), hi = __fmul_rn(__uint_as_float(w[j] & 0xffff0000u), rstd);
                    if (p.norm_hf) { lo = bf16r(lo); hi = bf16r(hi); }
                    o[j] = sk_bf2(__floats2bfloat162_rn(__fmul_rn(lo, __uint_as_float(gw[j] << 16)), __fmul_rn(hi, __uint_as_float(gw[j] & 0xffff0000u))));
                }
                stage_item(make_uint4(o[0], o[1], o[2], o[3]), tk, tid + u * (RB_WARPS * 32), true);
            }
            __syncthreads();                                                       // nred is reused by the next token
        }
    } else {
        // SB vectors per thread and round trip to L2: staging is a chain of such round trips (16 tokens of K = 4096 are
        // 32 vectors per thread)
        constexpr int SB = MT == 2 ? 8 : 4;
        const int kw_per_tok = NC4 ? 512 : p.K / 8, items = p.M * kw_per_tok;
        for (int base = 0; base < items; base += SB * RB_WARPS * 32) {
            uint4 v[SB];
            int tok[SB], kw[SB];
            bool on[SB];
#pragma unroll
            for (int h = 0; h < SB; ++h) {                // all loads first
                const int idx = base + h * RB_WARPS * 32 + tid;
                on[h] = idx < items;
                tok[h] = on[h] ? idx / kw_per_tok : 0; kw[h] = on[h] ? idx - tok[h] * kw_per_tok : 0;
                v[h] = on[h] ? reinterpret_cast<const uint4*>(p.x + (size_t)tok[h] * p.K)[kw[h]] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int h = 0; h < SB; ++h) stage_item(v[h], tok[h], kw[h], on[h]);
        }
    }
    __syncthreads();
    if constexpr (mma_sums) {
        const uint32_t ones[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
        for (int gi = 0; gi < n_groups; ++gi) {
            float sacc[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) sacc[m][0] = sacc[m][1] = sacc[m][2] = sacc[m][3] = 0.0f;
#pragma unroll
            for (int c = 0; c < GC; ++c)
#pragma unroll
                for (int w = 0; w < 4; ++w)
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint4 f = xs[(size_t)xrow[m] * x_stride + ((g_begin + gi) * GC + c) * 16 + w * 4 + t];
                        mma_16816(sacc[m], ones, f.x, f.y);
                        mma_16816(sacc[m], ones, f.z, f.w);
                    }
            if (g == 0) {                                 // every row of the D fragment holds the same sums
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    *reinterpret_cast<float2*>(&sxs[(g_begin + gi) * (8 * MT) + m * 8 + 2 * t]) = make_float2(sacc[m][0], sacc[m][1]);
            }
        }
        __syncwarp();                                     // a warp reads only the sums of its own groups
    }

    int buf = 0;
    // NC4: per-warp bases of the staged tokens and token sums (everything else is a compile-time offset)
    const uint4* xbase[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) xbase[m] = xs + (size_t)xrow[m] * x_stride + g_begin * 16 + t;
    const float* sxbase = sxs + g_begin * (8 * MT) + 2 * t;
    for (; blk < n_blocks; blk += gridDim.x) {
        const int nblk = blk + (int)gridDim.x;
        const bool has_next = nblk < n_blocks;
        const int na_row = has_next ? row_of(nblk, 0) : ra, nb_row = has_next ? row_of(nblk, 1) : rb;
        const uint4 *na = wptr(na_row), *nb = wptr(nb_row);
        float tot[MT][4], acc[MT][2][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) { tot[m][i] = acc[m][0][i] = acc[m][1][i] = 0.0f; }
        if constexpr (NC4) {
            uint2 ns4a = s4a, nz4a = z4a, ns4b = s4b, nz4b = z4b;
            if (has_next) { ns4a = load_s4(na_row); nz4a = load_z4(na_row); ns4b = load_s4(nb_row); nz4b = load_z4(nb_row); }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint4 ca = qa[u], cq = qb[u];
                if (has_next) { qa[u] = __ldg(na + u * 4); qb[u] = __ldg(nb + u * 4); }
                const uint32_t wsa[4] = {ca.x, ca.y, ca.z, ca.w}, wsb[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    LQ_WORD_FRAGS(wsa[w], wsb[w]);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint4 f = xbase[m][u * 16 + w * 4];
                        if (w == 0) {
                            mma_s_start(acc[m][0], a00, a01, a02, a03, f.x, f.y);
                            mma_s_start(acc[m][1], a10, a11, a12, a13, f.z, f.w);
                        } else {
                            mma_s(acc[m][0], a00, a01, a02, a03, f.x, f.y);
                            mma_s(acc[m][1], a10, a11, a12, a13, f.z, f.w);
                        }
                    }
                }
                // group u of the slice: bf16 bits (u & 1 ? high : low) half of word (u >> 1) of the packed loads
                const uint32_t sw_a = u < 2 ? s4a.x : s4a.y, zw_a = u < 2 ? z4a.x : z4a.y;
                const uint32_t sw_b = u < 2 ? s4b.x : s4b.y, zw_b = u < 2 ? z4b.x : z4b.y;
                const float s_a = __uint_as_float((u & 1) ? (sw_a & 0xffff0000u) : (sw_a << 16));
                const float z_a = __uint_as_float((u & 1) ? (zw_a & 0xffff0000u) : (zw_a << 16)) + 128.0f;
                const float s_b = __uint_as_float((u & 1) ? (sw_b & 0xffff0000u) : (sw_b << 16));
                const float z_b = __uint_as_float((u & 1) ? (zw_b & 0xffff0000u) : (zw_b << 16)) + 128.0f;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float2 sx = *reinterpret_cast<const float2*>(sxbase + u * (8 * MT) + m * 8);
                    tot[m][0] = fmaf(s_a, (acc[m][0][0] + acc[m][1][0]) - z_a * sx.x, tot[m][0]);
                    tot[m][1] = fmaf(s_a, (acc[m][0][1] + acc[m][1][1]) - z_a * sx.y, tot[m][1]);
                    tot[m][2] = fmaf(s_b, (acc[m][0][2] + acc[m][1][2]) - z_b * sx.x, tot[m][2]);
                    tot[m][3] = fmaf(s_b, (acc[m][0][3] + acc[m][1][3]) - z_b * sx.y, tot[m][3]);
                }
            }
            s4a = ns4a; z4a = nz4a; s4b = ns4b; z4b = nz4b;
        }
        if constexpr (NCH > 4) {
            // group parameters of this block and the next at constant offsets from one pointer per row and array
            const unsigned short *csa = sc_all + (size_t)ra * gpr + g_begin, *cza = zp_all + (size_t)ra * gpr + g_begin;
            const unsigned short *csb = sc_all + (size_t)rb * gpr + g_begin, *czb = zp_all + (size_t)rb * gpr + g_begin;
            const unsigned short *nsa = sc_all + (size_t)na_row * gpr + g_begin, *nza = zp_all + (size_t)na_row * gpr + g_begin;
            const unsigned short *nsb = sc_all + (size_t)nb_row * gpr + g_begin, *nzb = zp_all + (size_t)nb_row * gpr + g_begin;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int u = c & 3;
                if (c < n_chunks) {
                    const uint4 ca = qa[u], cq = qb[u];
                    sz_a = sza[u]; sz_b = szb[u];
                    if (c + 4 < n_chunks) {
                        qa[u] = __ldg(wa + (c + 4) * 4); qb[u] = __ldg(wb + (c + 4) * 4);
                        sza[u] = (uint32_t)__ldg(csa + c + 4) | ((uint32_t)__ldg(cza + c + 4) << 16);
                        szb[u] = (uint32_t)__ldg(csb + c + 4) | ((uint32_t)__ldg(czb + c + 4) << 16);
                    } else if (has_next) {                                           // slot u of the next row block
                        qa[u] = __ldg(na + u * 4); qb[u] = __ldg(nb + u * 4);
                        sza[u] = (uint32_t)__ldg(nsa + u) | ((uint32_t)__ldg(nza + u) << 16);
                        szb[u] = (uint32_t)__ldg(nsb + u) | ((uint32_t)__ldg(nzb + u) << 16);
                    }
                    const uint32_t wsa[4] = {ca.x, ca.y, ca.z, ca.w}, wsb[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        LQ_WORD_FRAGS(wsa[w], wsb[w]);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const uint4 f = xbase[m][c * 16 + w * 4];
                            if (w == 0) {
                                mma_s_start(acc[m][0], a00, a01, a02, a03, f.x, f.y);
                                mma_s_start(acc[m][1], a10, a11, a12, a13, f.z, f.w);
                            } else {
                                mma_s(acc[m][0], a00, a01, a02, a03, f.x, f.y);
                                mma_s(acc[m][1], a10, a11, a12, a13, f.z, f.w);
                            }
                        }
                    }
                    const float s_a = __uint_as_float(sz_a << 16), z_a = __uint_as_float(sz_a & 0xffff0000u) + 128.0f;
                    const float s_b = __uint_as_float(sz_b << 16), z_b = __uint_as_float(sz_b & 0xffff0000u) + 128.0f;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float2 sx = *reinterpret_cast<const float2*>(sxbase + c * (8 * MT) + m * 8);
                        tot[m][0] = fmaf(s_a, (acc[m][0][0] + acc[m][1][0]) - z_a * sx.x, tot[m][0]);
                        tot[m][1] = fmaf(s_a, (acc[m][0][1] + acc[m][1][1]) - z_a * sx.y, tot[m][1]);
                        tot[m][2] = fmaf(s_b, (acc[m][0][2] + acc[m][1][2]) - z_b * sx.x, tot[m][2]);
                        tot[m][3] = fmaf(s_b, (acc[m][0][3] + acc[m][1][3]) - z_b * sx.y, tot[m][3]);
                    }
                }
            }
        }
        int grp = 0;
        for (int cb = 0; NCH == 0 && cb < n_chunks; cb += PF) {
#pragma unroll
            for (int u = 0; u < PF; ++u) {
                const int c = cb + u;
                if (c < n_chunks) {
                    const uint4 ca = qa[u], cq = qb[u];
                    if (u % GC == 0) { sz_a = sza[u]; sz_b = szb[u]; }
                    if (c + PF < n_chunks) {
                        qa[u] = __ldg(wa + (c + PF) * 4); qb[u] = __ldg(wb + (c + PF) * 4);
                        if (u % GC == 0) { sza[u] = load_sz(ra, (c + PF) / GC); szb[u] = load_sz(rb, (c + PF) / GC); }
                    } else if (has_next) {                                                          // slot u of the next row block
                        qa[u] = __ldg(na + u * 4); qb[u] = __ldg(nb + u * 4);
                        if (u % GC == 0) { sza[u] = load_sz(na_row, u / GC); szb[u] = load_sz(nb_row, u / GC); }
                    }
                    const uint32_t wsa[4] = {ca.x, ca.y, ca.z, ca.w}, wsb[4] = {cq.x, cq.y, cq.z, cq.w};
                    const int cg = g_begin * GC + c;                                              // chunk index within the row
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        LQ_WORD_FRAGS(wsa[w], wsb[w]);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const uint4 f = xs[(size_t)xrow[m] * x_stride + cg * 16 + w * 4 + t];
                            if (w == 0 && u % GC == 0) {            // first word of a group: no accumulator input
                                mma_s_start(acc[m][0], a00, a01, a02, a03, f.x, f.y);
                                mma_s_start(acc[m][1], a10, a11, a12, a13, f.z, f.w);
                            } else {
                                mma_s(acc[m][0], a00, a01, a02, a03, f.x, f.y);
                                mma_s(acc[m][1], a10, a11, a12, a13, f.z, f.w);
                            }
                        }
                    }
                    if ((u + 1) % GC == 0) {
                        // fold the group: s * (sum x (128 + q) - (128 + z) * sum x), then rotate the group parameters
                        const float s_a = __uint_as_float(sz_a << 16), z_a = __uint_as_float(sz_a & 0xffff0000u) + 128.0f;
                        const float s_b = __uint_as_float(sz_b << 16), z_b = __uint_as_float(sz_b & 0xffff0000u) + 128.0f;
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const float2 sx = *reinterpret_cast<const float2*>(&sxs[(g_begin + grp) * (8 * MT) + m * 8 + 2 * t]);
                            tot[m][0] = fmaf(s_a, (acc[m][0][0] + acc[m][1][0]) - z_a * sx.x, tot[m][0]);
                            tot[m][1] = fmaf(s_a, (acc[m][0][1] + acc[m][1][1]) - z_a * sx.y, tot[m][1]);
                            tot[m][2] = fmaf(s_b, (acc[m][0][2] + acc[m][1][2]) - z_b * sx.x, tot[m][2]);
                            tot[m][3] = fmaf(s_b, (acc[m][0][3] + acc[m][1][3]) - z_b * sx.y, tot[m][3]);
                        }
                        ++grp;
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m)
            *reinterpret_cast<float4*>(&red[buf][warp][m][lane * 4]) = make_float4(tot[m][0], tot[m][1], tot[m][2], tot[m][3]);
        __syncthreads();      // one barrier per row block: the other buffer is rewritten only after the next barrier
        // D fragment: d0,d1 = (row g, tokens 2t, 2t+1); d2,d3 = (row g+8, same tokens)
        for (int j = tid; j < MT * 128; j += RB_WARPS * 32) {
            const int m = j >> 7, idx = j & 127, ln = idx >> 2, i = idx & 3;
            const int tok = m * 8 + 2 * (ln & 3) + (i & 1);
            if (pair) {                                        // d0,d1 = gate[f], d2,d3 = up[f] of the same tokens
                const int f = blk * 8 + (ln >> 2);
                if (i >= 2 || f >= p.N || tok >= p.M) continue;
                float ag = 0.0f, au = 0.0f;
#pragma unroll
                for (int w = 0; w < RB_WARPS; ++w) { ag = __fadd_rn(ag, red[buf][w][m][idx]); au = __fadd_rn(au, red[buf][w][m][idx + 2]); }
                if (p.rope_hd) { rope_store(p, blk, ln >> 2, tok, bf16r(ag), bf16r(au)); continue; }
                p.out[(size_t)tok * p.N + f] = __float2bfloat16_rn(silu_mul_bf16(bf16r(ag), bf16r(au), p.hf_rounding));
                continue;
            }
            const int row = blk * 16 + (ln >> 2) + ((i >= 2) ? 8 : 0);
            if (row >= p.N || tok >= p.M) continue;
            float a = 0.0f;
#pragma unroll
            for (int w = 0; w < RB_WARPS; ++w) a = __fadd_rn(a, red[buf][w][m][idx]);
            const float f = bf16r(a);
            p.out[(size_t)tok * p.N + row] = __float2bfloat16_rn(p.bias ? __fadd_rn(f, __bfloat162float(p.bias[row])) : f);
        }
        buf ^= 1;
        ra = na_row; rb = nb_row; wa = na; wb = nb;
    }
}

bool skinny_norm_supported(int64_t M, int64_t K, int group) {
    return M >= 1 && M <= 2 && K == 4096 && group == 128 && LQ_GEMV_PF == 4 && !getenv("LQ_SKINNY_NO_NC4") && !getenv("LQ_SKINNY_NO_STREAM");
}
bool skinny_rows_supported(int64_t K, int group) { return (group == 128 || group == 256) && K % group == 0; }

// every warp of the streaming kernel needs at least two whole groups of the row
static bool skinny_stream_supported(int64_t K, int group) {
    if (!skinny_rows_supported(K, group) || getenv("LQ_SKINNY_NO_STREAM")) return false;
    const int gpr = (int)(K / group), gper = (gpr + RB_WARPS - 1) / RB_WARPS;
    return gpr - (RB_WARPS - 1) * gper >= 2;
}

template <int MT, int GC, int NCH = 0, bool NORM = false>
static int launch_skinny_stream_v(const SkinnyParams& p, int x_stride, size_t smem, unsigned grid, cudaStream_t st) {
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return LQ_EUNSUPPORTED;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_skinny_stream<MT, GC, NCH, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (MT == 2 ? 144 : 96) * 1024);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(k_skinny_stream)"); return LQ_ECUDA; }
        attr_done[dev] = true;
    }
    launch_pdl(k_skinny_stream<MT, GC, NCH, NORM>, dim3(grid), RB_WARPS * 32, smem, st, p, x_stride);
    return check_launch("k_skinny_stream");
}

// token rows 64 bytes apart modulo 128: conflict-free 16-byte reads of two tokens by a quarter warp
static int skinny_x_stride(int K) { const int kw = K / 8; return kw + ((4 - (kw & 7)) & 7); }
static size_t skinny_stream_smem(int M, int K, int group) {
    return (size_t)M * skinny_x_stride(K) * 16 + (size_t)(K / group) * 8 * (M <= 8 ? 1 : 2) * sizeof(float);
}

static int launch_skinny_stream(const SkinnyParams& p, cudaStream_t st) {
    const int mt = p.M <= 8 ? 1 : 2, gc = p.group / RB_CHUNK;
    const int x_stride = skinny_x_stride(p.K);
    const size_t smem = skinny_stream_smem(p.M, p.K, p.group);
    const int rpb = p.pair_stride > 0 ? 8 : 16;
    const int n_blocks = (p.N + rpb - 1) / rpb;
    const unsigned grid = (unsigned)std::min(n_blocks, (mt == 2 ? 1 : LQ_GEMV_MINB) * sm_count());   // 9-16 tokens: one CTA per SM
    // K = 4096 with groups of 128: the written-out loop (scales / zeros are read as 8-byte words there)
    const bool nc4 = gc == 1 && p.K == 4096 && LQ_GEMV_PF == 4 && !getenv("LQ_SKINNY_NO_NC4") &&
                     (reinterpret_cast<uintptr_t>(p.scales) & 7) == 0 && (reinterpret_cast<uintptr_t>(p.zeros) & 7) == 0;
    if (p.norm_gamma) {                             // fused-norm staging exists for the written-out K = 4096 loop, up to 8 tokens
        if (!nc4 || mt != 1) return LQ_EUNSUPPORTED;
        return launch_skinny_stream_v<1, 1, 4, true>(p, x_stride, smem, grid, st);
    }
    if (nc4) return mt == 1 ? launch_skinny_stream_v<1, 1, 4>(p, x_stride, smem, grid, st) : launch_skinny_stream_v<2, 1, 4>(p, x_stride, smem, grid, st);
    if (gc == 1 && p.K == 11008 && LQ_GEMV_PF == 4 && !getenv("LQ_SKINNY_NO_NC4"))      // eleven chunks per warp, written out
        return mt == 1 ? launch_skinny_stream_v<1, 1, 11>(p, x_stride, smem, grid, st) : launch_skinny_stream_v<2, 1, 11>(p, x_stride, smem, grid, st);
    if (mt == 1) return gc == 1 ? launch_skinny_stream_v<1, 1>(p, x_stride, smem, grid, st) : launch_skinny_stream_v<1, 2>(p, x_stride, smem, grid, st);
    return gc == 1 ? launch_skinny_stream_v<2, 1>(p, x_stride, smem, grid, st) : launch_skinny_stream_v<2, 2>(p, x_stride, smem, grid, st);
}

int launch_skinny_rows(const SkinnyParams& p, cudaStream_t st) {
    if (!skinny_rows_supported(p.K, p.group)) return LQ_EUNSUPPORTED;
    // two CTAs per SM must fit: staged tokens + sums + 8-16 KB of static shared memory each
    // 9-16 tokens at K = 4096: the same kernel with one CTA per SM (its 16 staged tokens take 130 KB); the row-block
    // kernel below re-reads every token from L2 in every CTA (128 KB per 32 KB of weights) and permutes it per use.
    // Staging the tokens is a fixed cost per CTA, so from three tokens on the kernel pays only for launches with many row
    // blocks per CTA (measured: the q|k|v and gate|up projections of the 7B shapes, not the 4096-row ones).
    const int n_row_blocks = (p.N + (p.pair_stride > 0 ? 8 : 16) - 1) / (p.pair_stride > 0 ? 8 : 16);
    const int wide_min = getenv("LQ_SKINNY_WIDE_MIN") ? atoi(getenv("LQ_SKINNY_WIDE_MIN")) : 768;
    const bool wide = p.M > 2 && p.K == 4096 && p.group == 128 && n_row_blocks >= wide_min && !getenv("LQ_SKINNY_NO_STREAM16");
    // One or two tokens: the streaming kernel when there are more row blocks than persistent CTAs; a launch of one row
    // block per CTA is the kernel below's case (measured at one token: 3.9 against 4.2 us for 4096 x 4096, 9.0 against
    // 11.2 us for the 11008 -> 4096 down projection).  A fused norm follows the same rule, so that it always computes
    // the bits of the two-launch sequence.
    const bool small = p.M <= 2 && n_row_blocks > LQ_GEMV_MINB * sm_count();
    if ((small || wide || getenv("LQ_SKINNY_STREAM_ALL")) && skinny_stream_supported(p.K, p.group) &&
        skinny_stream_smem(p.M, p.K, p.group) <= (size_t)(p.M > 8 ? 144 : 96) * 1024)
        return launch_skinny_stream(p, st);
    if (p.norm_gamma) return LQ_EUNSUPPORTED;       // the fused-norm staging exists in the streaming kernel only
    const int rpb = p.pair_stride > 0 ? 8 : 16;
    const unsigned grid = (unsigned)((p.N + rpb - 1) / rpb);
    const bool g128 = p.group == 128;
    // K = 4096 with groups of 128: the written-out loop (scales / zeros are read as 8-byte words there)
    const bool nc4 = g128 && p.K == 4096 && !getenv("LQ_SKINNY_NO_NC4") &&
                     (reinterpret_cast<uintptr_t>(p.scales) & 7) == 0 && (reinterpret_cast<uintptr_t>(p.zeros) & 7) == 0;
    if (nc4) {
        if (p.M <= 8) launch_pdl(k_skinny_rows<1, 1, 4>, dim3(grid), RB_WARPS * 32, 0, st, p);
        else launch_pdl(k_skinny_rows<2, 1, 4>, dim3(grid), RB_WARPS * 32, 0, st, p);
        return check_launch("k_skinny_rows");
    }
    if (g128 && p.K == 11008 && !getenv("LQ_SKINNY_NO_NC4")) {          // eleven chunks per warp, written out
        if (p.M <= 8) launch_pdl(k_skinny_rows<1, 1, 11>, dim3(grid), RB_WARPS * 32, 0, st, p);
        else launch_pdl(k_skinny_rows<2, 1, 11>, dim3(grid), RB_WARPS * 32, 0, st, p);
        return check_launch("k_skinny_rows");
    }
    if (p.M <= 8) { if (g128) launch_pdl(k_skinny_rows<1, 1>, dim3(grid), RB_WARPS * 32, 0, st, p); else launch_pdl(k_skinny_rows<1, 2>, dim3(grid), RB_WARPS * 32, 0, st, p); }
    else { if (g128) launch_pdl(k_skinny_rows<2, 1>, dim3(grid), RB_WARPS * 32, 0, st, p); else launch_pdl(k_skinny_rows<2, 2>, dim3(grid), RB_WARPS * 32, 0, st, p); }
    return check_launch("k_skinny_rows");
}

int skinny_chunks_per_split(int64_t N, int64_t K, int* splits_out) {
    const int n_blocks = (int)((N + SK_ROWS - 1) / SK_ROWS);
    const int chunks_total = (int)(K / SK_CHUNK);
    const int gc = 4;                                               // slices are multiples of 256 k: whole groups of 64/128/256
    int splits = (4 * sm_count() + n_blocks - 1) / n_blocks;     // ~4 CTAs per SM in flight
    if (splits > chunks_total / 4) splits = chunks_total / 4;    // at least 4 chunks (256 k) per CTA
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
    int per = (chunks_total + splits - 1) / splits;
    per = (per + gc - 1) / gc * gc;                                 // a slice holds whole quantization groups
    *splits_out = (chunks_total + per - 1) / per;
    return per;
}

int launch_skinny_fwd(const SkinnyParams& p, cudaStream_t st) {
    const int mt = p.M <= 8 ? 1 : 2;
    const size_t smem = (size_t)mt * 8 * (p.chunks_per_split * SK_CHUNK + SK_XPAD) * sizeof(__nv_bfloat16);
    if (smem > 200 * 1024) return LQ_EUNSUPPORTED;
    dim3 grid((unsigned)((p.N + SK_ROWS - 1) / SK_ROWS), (unsigned)p.splits);
    static bool attr_done[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev][mt - 1]) {
        cudaError_t e = mt == 1 ? cudaFuncSetAttribute(k_skinny_fwd<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                : cudaFuncSetAttribute(k_skinny_fwd<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(k_skinny_fwd)"); return LQ_ECUDA; }
        attr_done[dev][mt - 1] = true;
    }
    if (mt == 1) k_skinny_fwd<1><<<grid, SK_THREADS, smem, st>>>(p);
    else k_skinny_fwd<2><<<grid, SK_THREADS, smem, st>>>(p);
    return check_launch("k_skinny_fwd");
}

}  // namespace lq
