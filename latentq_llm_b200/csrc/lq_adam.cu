// Fused optimizer step of the latent fine-tune path: one HBM pass per quantized weight instead of the ~40
// tensor-op passes of MyAdam.update_step (utils/quant.py:1052-1148), and one launch for all the small dense
// parameters.  Every intermediate is rounded where the reference's torch ops round it (each op computes in fp32
// and stores in the tensor dtype), so codes, residual words and optimizer states come out bit-identical to the
// op-by-op route.
//
// Where torch's CUDA functors are single expressions (`a + alpha * b`, `a + alpha * (b / c)`), nvcc contracts the
// multiply-add into an FMA in torch's own build; the same contraction is spelled out here with __fmaf_rn
// (checked on the GPU against torch's add_/addcmul_/addcdiv_ on 2^24-element bf16 tensors: the separately
// rounded forms of add_(alpha) and addcdiv_ differ from torch in a few elements per million, the fused ones never).
#include <cstdlib>

#include "lq_requant.cuh"

namespace lq {

struct AdamParams {
    RequantParams rq;
    const void* grad; int grad_dtype;
    uint8_t* st1; float* sc1; float* tm1;
    uint8_t* st2; float* sc2; float* tm2;
    int opt_shift;                 // log2(elements per optimizer-state block): 11 or 7
    int64_t n_tiles;               // tiles of 256 words
    lq_adam_hyper h;
};

// m <- m*b1 ; m <- m + (1-b1)*g ; v <- v*b2 ; v <- v + (1-b2)*(g*g) ; d <- sqrt(v) ; d <- d + eps ; each stored in
// the chain dtype (utils/quant.py:1098-1101).  Returns m and d = sqrt(v)+eps.
template <bool BF>
__device__ __forceinline__ void adam_moments(const lq_adam_hyper& h, float g, float& m, float& v_to_d) {
    m = rb<BF>(__fmul_rn(m, h.beta1));
    m = rb<BF>(__fmaf_rn(h.one_minus_beta1, g, m));
    float v = rb<BF>(__fmul_rn(v_to_d, h.beta2));
    v = rb<BF>(__fmaf_rn(h.one_minus_beta2, __fmul_rn(g, g), v));
    float d = rb<BF>(__fsqrt_rn(v));
    v_to_d = rb<BF>(__fadd_rn(d, h.eps));
}
// p <- p + (-step_size) * (m / d)   (addcdiv_, utils/quant.py:1105)
template <bool BF>
__device__ __forceinline__ float adam_apply(const lq_adam_hyper& h, float p, float m, float d) {
    return rb<BF>(__fmaf_rn(h.neg_step_size, __fdiv_rn(m, d), p));
}

__device__ __forceinline__ uint2 opt8_encode8(const float (&x)[8], float mx, float s) {
    const float rs = __frcp_rn(s);
    const bool ok = fastdiv_ok_scale(s);
    uint32_t b[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float t = rne(div_rn(__fsub_rn(mx, x[k]), s, rs, ok));
        t = fminf(fmaxf(t, 0.0f), 255.0f);
        b[k] = f2bits(t) & 0xffu;
    }
    uint2 o;
    o.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    o.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
    return o;
}

// One thread per word of 8 elements; a CTA covers 256 words = one 2048-element optimizer-state block, or sixteen
// 128-element blocks (16 lanes each).
template <int WBITS, int CODEC, int DITHER, bool BF>
__global__ void __launch_bounds__(256) k_adam_quant(const AdamParams p) {
    __shared__ float s_red[4][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
        const int64_t w = tile * 256 + tid;
        const bool active = w < p.rq.n_words;
        const int64_t e0 = w * 8;
        float lat[8], m[8], d[8];
        float s = 1.0f, z = 0.0f;
        float mn1 = INFINITY, mx1 = -INFINITY, mn2 = INFINITY, mx2 = -INFINITY;
        int64_t ob = 0;
        if (active) {
            const int64_t g = p.rq.group_shift >= 0 ? (e0 >> p.rq.group_shift) : (e0 / p.rq.group);
            s = load1(p.rq.scales, p.rq.qp_dtype, g);
            z = (WBITS == 4) ? load1(p.rq.zeros, p.rq.qp_dtype, g) : 0.0f;
            ob = e0 >> p.opt_shift;
            const float s1 = p.sc1[ob], t1 = p.tm1[ob], s2 = p.sc2[ob], t2 = p.tm2[ob];   // rewritten below: plain loads
            const uint2 q1 = *reinterpret_cast<const uint2*>(p.st1 + e0);
            const uint2 q2 = *reinterpret_cast<const uint2*>(p.st2 + e0);
            float gr[8];
            load8(p.grad, p.grad_dtype, e0, gr);
            latent_load<WBITS, CODEC, BF>(p.rq, w, s, z, lat);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float c1 = u2f(((k < 4 ? q1.x : q1.y) >> (8 * (k & 3))) & 0xffu);
                const float c2 = u2f(((k < 4 ? q2.x : q2.y) >> (8 * (k & 3))) & 0xffu);
                m[k] = rb<BF>(__fsub_rn(t1, __fmul_rn(c1, s1)));           // DeQfunc_8bit_opt(...).to(dtype)
                const float r2 = __fsub_rn(t2, __fmul_rn(c2, s2));
                d[k] = rb<BF>(__fmul_rn(r2, r2));                          // (s2 * s2).to(dtype)
                adam_moments<BF>(p.h, gr[k], m[k], d[k]);
                lat[k] = adam_apply<BF>(p.h, lat[k], m[k], d[k]);
                mn1 = fminf(mn1, m[k]); mx1 = fmaxf(mx1, m[k]);
                mn2 = fminf(mn2, d[k]); mx2 = fmaxf(mx2, d[k]);
            }
        }
        // min/max over the optimizer-state block: 16 lanes, then (2048-element blocks) the whole CTA
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            mn1 = fminf(mn1, __shfl_xor_sync(0xffffffffu, mn1, o)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            mn2 = fminf(mn2, __shfl_xor_sync(0xffffffffu, mn2, o)); mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, o));
        }
        if (p.opt_shift == 11) {
            mn1 = fminf(mn1, __shfl_xor_sync(0xffffffffu, mn1, 16)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 16));
            mn2 = fminf(mn2, __shfl_xor_sync(0xffffffffu, mn2, 16)); mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 16));
            __syncthreads();                                               // previous tile's readers are done
            if (lane == 0) { s_red[0][warp] = mn1; s_red[1][warp] = mx1; s_red[2][warp] = mn2; s_red[3][warp] = mx2; }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                mn1 = fminf(mn1, s_red[0][i]); mx1 = fmaxf(mx1, s_red[1][i]);
                mn2 = fminf(mn2, s_red[2][i]); mx2 = fmaxf(mx2, s_red[3][i]);
            }
        }
        if (active) {
            const float ns1 = __fadd_rn(__fdiv_rn(__fsub_rn(mx1, mn1), 255.0f), 1e-10f);
            const float ns2 = __fadd_rn(__fdiv_rn(__fsub_rn(mx2, mn2), 255.0f), 1e-10f);
            *reinterpret_cast<uint2*>(p.st1 + e0) = opt8_encode8(m, mx1, ns1);
            *reinterpret_cast<uint2*>(p.st2 + e0) = opt8_encode8(d, mx2, ns2);
            const bool leader = p.opt_shift == 11 ? (tid == 0) : ((tid & 15) == 0);
            if (leader) { p.sc1[ob] = ns1; p.tm1[ob] = mx1; p.sc2[ob] = ns2; p.tm2[ob] = mx2; }
            latent_store<WBITS, CODEC, DITHER, BF>(p.rq, w, s, z, lat);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Fast variant of the production configuration (bf16 chain, bf16 qparams and gradient, 3-fold codec, hash dither, group a
// power of two >= 8): packed bf16x2 reconstruction of the latent weights with the residual decode from a 256-entry table,
// bf16 roundings as packed conversions (two values per instruction), and everything after Z = w/scale + zero from the
// 64 KB table of the requantize fast path.  Same results as k_adam_a16w4, bit for bit; a word whose Z leaves the table's
// range (|Z| >= 64, non-finite) is encoded by the generic chain.
// ---------------------------------------------------------------------------------------------------------------
constexpr int ADAM_TRES_REPL = 8;
constexpr int ADAM_FAST_SMEM = ENCZ_TABLE_ENTRIES + 256 * ADAM_TRES_REPL * 4;

__device__ __forceinline__ void rb2(float a, float b, float& ra, float& rbv) {       // bf16 roundings of two values, one conversion
    const __nv_bfloat162 q = __floats2bfloat162_rn(a, b);
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&q);
    ra = __uint_as_float(u << 16); rbv = __uint_as_float(u & 0xffff0000u);
}

template <bool USE_RES>
__global__ void __launch_bounds__(256, 3) k_adam_a16w4_fast(const AdamParams p, const int enc_slot) {
    extern __shared__ __align__(16) uint8_t asm_[];
    uint8_t* encz = asm_;
    uint32_t* tres = reinterpret_cast<uint32_t*>(asm_ + ENCZ_TABLE_ENTRIES);
    __shared__ float s_red[4][8];
    {
        const uint4* src = reinterpret_cast<const uint4*>(g_encz_table[enc_slot]);
        uint4* dst = reinterpret_cast<uint4*>(encz);
        for (int i = threadIdx.x; i < ENCZ_TABLE_ENTRIES / 16; i += 256) dst[i] = __ldg(src + i);
        for (int b = threadIdx.x; b < 256; b += 256) {
            const uint32_t lo = f32_to_bf16_bits(bf16r(res3_decode((uint32_t)b >> 4, p.rq.dec)));
            const uint32_t hi = f32_to_bf16_bits(bf16r(res3_decode((uint32_t)b & 15u, p.rq.dec)));
            for (int r = 0; r < ADAM_TRES_REPL; ++r) tres[b * ADAM_TRES_REPL + r] = lo | (hi << 16);
        }
    }
    __syncthreads();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t tres_lane = tid & (ADAM_TRES_REPL - 1);
    const unsigned short* scales = reinterpret_cast<const unsigned short*>(p.rq.scales);
    const unsigned short* zeros = reinterpret_cast<const unsigned short*>(p.rq.zeros);
    const uint32_t n_words = (uint32_t)p.rq.n_words;
    const int gsh = p.rq.group_shift - 3;                     // word index -> group index
    const int osh = p.opt_shift - 3;                          // word index -> optimizer-state block
    const uint32_t c128u = 0x43004300u;
    for (uint32_t tile = blockIdx.x; tile < (uint32_t)p.n_tiles; tile += gridDim.x) {
        const uint32_t w = tile * 256u + (uint32_t)tid;
        const bool active = w < n_words;
        float lat[8], m[8], d[8];
        float sf = 1.0f;
        uint32_t zb = 0u, ob = 0u;
        float mn1 = INFINITY, mx1 = -INFINITY, mn2 = INFINITY, mx2 = -INFINITY;
        if (active) {
            const uint32_t g = w >> gsh;
            const uint32_t sb = __ldg(scales + g);
            zb = __ldg(zeros + g);
            ob = w >> osh;
            const float s1 = p.sc1[ob], t1 = p.tm1[ob], s2f = p.sc2[ob], t2 = p.tm2[ob];
            const uint2 q1 = *reinterpret_cast<const uint2*>(p.st1 + (size_t)w * 8);
            const uint2 q2 = *reinterpret_cast<const uint2*>(p.st2 + (size_t)w * 8);
            const uint4 gv = __ldg(reinterpret_cast<const uint4*>(p.grad) + w);
            const uint32_t pk = __ldg(reinterpret_cast<const uint32_t*>(p.rq.codes_in) + w);
            uint32_t rw = 0u;
            if (USE_RES) rw = (uint32_t)__ldg(p.rq.words_in + w);
            sf = __uint_as_float(sb << 16);
            // latent weights: bf16((q - z) * s) (+ bf16(bf16(res * s) + that)), packed
            const uint32_t s2u = sb * 0x00010001u, z2u = zb * 0x00010001u;
            const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&s2u);
            const __nv_bfloat162 z128 = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&z2u), *reinterpret_cast<const __nv_bfloat162*>(&c128u));
            const uint32_t lo_n = pk & 0x0F0F0F0Fu, hi_n = (pk >> 4) & 0x0F0F0F0Fu;
            const uint32_t c03 = __byte_perm(hi_n, lo_n, 0x5140), c47 = __byte_perm(hi_n, lo_n, 0x7362);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pair = __byte_perm((j < 2) ? c03 : c47, 0x43434343u, (j & 1) ? 0x4342 : 0x4140);
                __nv_bfloat162 v = __hmul2_rn(__hsub2_rn(*reinterpret_cast<const __nv_bfloat162*>(&pair), z128), s2);
                if (USE_RES) {
                    const uint32_t b = (rw >> (24 - 8 * j)) & 0xffu;
                    const uint32_t tr = tres[b * ADAM_TRES_REPL + tres_lane];
                    v = __hadd2_rn(__hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&tr), s2), v);
                }
                const uint32_t vu = *reinterpret_cast<const uint32_t*>(&v);
                lat[2 * j] = __uint_as_float(vu << 16); lat[2 * j + 1] = __uint_as_float(vu & 0xffff0000u);
                // the two elements of the pair through the optimizer chain (every intermediate rounded to bf16)
                const int k0 = 2 * j, k1 = 2 * j + 1;
                const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
                const float c10 = u2f(((k0 < 4 ? q1.x : q1.y) >> (8 * (k0 & 3))) & 0xffu), c11 = u2f(((k1 < 4 ? q1.x : q1.y) >> (8 * (k1 & 3))) & 0xffu);
                const float c20 = u2f(((k0 < 4 ? q2.x : q2.y) >> (8 * (k0 & 3))) & 0xffu), c21 = u2f(((k1 < 4 ? q2.x : q2.y) >> (8 * (k1 & 3))) & 0xffu);
                float m0, m1, v0, v1, t0, t1v;
                rb2(__fsub_rn(t1, __fmul_rn(c10, s1)), __fsub_rn(t1, __fmul_rn(c11, s1)), m0, m1);       // DeQfunc_8bit_opt(...).to(bf16)
                const float r20 = __fsub_rn(t2, __fmul_rn(c20, s2f)), r21 = __fsub_rn(t2, __fmul_rn(c21, s2f));
                rb2(__fmul_rn(r20, r20), __fmul_rn(r21, r21), v0, v1);                                   // (s2 * s2).to(bf16)
                rb2(__fmul_rn(m0, p.h.beta1), __fmul_rn(m1, p.h.beta1), m0, m1);
                rb2(__fmaf_rn(p.h.one_minus_beta1, g0, m0), __fmaf_rn(p.h.one_minus_beta1, g1, m1), m0, m1);
                rb2(__fmul_rn(v0, p.h.beta2), __fmul_rn(v1, p.h.beta2), v0, v1);
                rb2(__fmaf_rn(p.h.one_minus_beta2, __fmul_rn(g0, g0), v0), __fmaf_rn(p.h.one_minus_beta2, __fmul_rn(g1, g1), v1), v0, v1);
                rb2(__fsqrt_rn(v0), __fsqrt_rn(v1), t0, t1v);
                rb2(__fadd_rn(t0, p.h.eps), __fadd_rn(t1v, p.h.eps), v0, v1);                            // sqrt(v) + eps
                rb2(__fmaf_rn(p.h.neg_step_size, __fdiv_rn(m0, v0), lat[k0]), __fmaf_rn(p.h.neg_step_size, __fdiv_rn(m1, v1), lat[k1]), lat[k0], lat[k1]);
                m[k0] = m0; m[k1] = m1; d[k0] = v0; d[k1] = v1;
                mn1 = fminf(mn1, fminf(m0, m1)); mx1 = fmaxf(mx1, fmaxf(m0, m1));
                mn2 = fminf(mn2, fminf(v0, v1)); mx2 = fmaxf(mx2, fmaxf(v0, v1));
            }
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            mn1 = fminf(mn1, __shfl_xor_sync(0xffffffffu, mn1, o)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
            mn2 = fminf(mn2, __shfl_xor_sync(0xffffffffu, mn2, o)); mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, o));
        }
        if (p.opt_shift == 11) {
            mn1 = fminf(mn1, __shfl_xor_sync(0xffffffffu, mn1, 16)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 16));
            mn2 = fminf(mn2, __shfl_xor_sync(0xffffffffu, mn2, 16)); mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 16));
            __syncthreads();
            if (lane == 0) { s_red[0][warp] = mn1; s_red[1][warp] = mx1; s_red[2][warp] = mn2; s_red[3][warp] = mx2; }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                mn1 = fminf(mn1, s_red[0][i]); mx1 = fmaxf(mx1, s_red[1][i]);
                mn2 = fminf(mn2, s_red[2][i]); mx2 = fmaxf(mx2, s_red[3][i]);
            }
        }
        if (active) {
            const float ns1 = __fadd_rn(__fdiv_rn(__fsub_rn(mx1, mn1), 255.0f), 1e-10f);
            const float ns2 = __fadd_rn(__fdiv_rn(__fsub_rn(mx2, mn2), 255.0f), 1e-10f);
            *reinterpret_cast<uint2*>(p.st1 + (size_t)w * 8) = opt8_encode8(m, mx1, ns1);
            *reinterpret_cast<uint2*>(p.st2 + (size_t)w * 8) = opt8_encode8(d, mx2, ns2);
            const bool leader = p.opt_shift == 11 ? (tid == 0) : ((tid & 15) == 0);
            if (leader) { p.sc1[ob] = ns1; p.tm1[ob] = mx1; p.sc2[ob] = ns2; p.tm2[ob] = mx2; }
            // requantize: Z = bf16(bf16(lat / s) + z), then one table byte per element
            const float rs = __frcp_rn(sf);
            const uint32_t z2u = zb * 0x00010001u;
            const __nv_bfloat162 z2 = *reinterpret_cast<const __nv_bfloat162*>(&z2u);
            uint32_t zbits[4], zmax = 0u;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 Zp = __hadd2_rn(__floats2bfloat162_rn(__fmul_rn(lat[2 * j], rs), __fmul_rn(lat[2 * j + 1], rs)), z2);
                zbits[j] = *reinterpret_cast<const uint32_t*>(&Zp);
                __nv_bfloat162 az = __habs2(Zp);
                if (j) az = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162*>(&zmax), az);        // NaN-propagating max of the magnitudes
                zmax = *reinterpret_cast<const uint32_t*>(&az);
            }
            const bool bad = (((zmax & 0x7fff7fffu) + 0x3d803d80u) & 0x80008000u) != 0u || !fastdiv_ok_scale(sf);
            if (__builtin_expect(bad, 0)) {
                const float z = __uint_as_float(zb << 16);
                latent_store<4, LQ_CODEC_THREEFOLD, LQ_DITHER_HASH, true>(p.rq, (int64_t)w, sf, z, lat);
            } else {
                uint32_t ev[4], od[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) { ev[j] = encz[zbits[j] & 0xffffu]; od[j] = encz[zbits[j] >> 16]; }
                const uint32_t e_even = __byte_perm(__byte_perm(ev[0], ev[1], 0x4040), __byte_perm(ev[2], ev[3], 0x4040), 0x5410);
                const uint32_t e_odd = __byte_perm(__byte_perm(od[0], od[1], 0x4040), __byte_perm(od[2], od[3], 0x4040), 0x5410);
                reinterpret_cast<uint32_t*>(p.rq.codes_out)[w] = (e_even & 0xF0F0F0F0u) | ((e_odd >> 4) & 0x0F0F0F0Fu);
                p.rq.words_out[w] = (int32_t)__byte_perm(((e_even << 4) & 0xF0F0F0F0u) | (e_odd & 0x0F0F0F0Fu), 0u, 0x0123);
            }
        }
    }
}

template <int WBITS, int CODEC, int DITHER>
static int launch_adam(const AdamParams& p, bool bf, cudaStream_t st) {
    const int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(p.n_tiles < cap ? p.n_tiles : cap);
    if (bf) k_adam_quant<WBITS, CODEC, DITHER, true><<<grid, 256, 0, st>>>(p);
    else k_adam_quant<WBITS, CODEC, DITHER, false><<<grid, 256, 0, st>>>(p);
    return check_launch("k_adam_quant");
}

// ---- the statistic behind the residual-curve refresh (utils/quant.py:1107-1111) ---------------------------------
// abs(exp_avg) / denom of the step ABOUT to be taken (the reference evaluates it after the moment update and before
// the requantize, whose curve level it may change), summed in fp32 over runs of 128 elements: 16 adjacent threads, fixed
// order.  Reads the gradient and both 8-bit states, writes only the sums.
template <bool BF>
__global__ void __launch_bounds__(256) k_adam_moment_stat(const AdamParams p, float* __restrict__ stat_out) {
    for (int64_t w = (int64_t)blockIdx.x * 256 + threadIdx.x; w < p.n_tiles * 256; w += (int64_t)gridDim.x * 256) {
        const bool active = w < p.rq.n_words;
        float t = 0.0f;
        if (active) {
            const int64_t e0 = w * 8, ob = e0 >> p.opt_shift;
            const float s1 = p.sc1[ob], t1 = p.tm1[ob], s2 = p.sc2[ob], t2 = p.tm2[ob];
            const uint2 q1 = *reinterpret_cast<const uint2*>(p.st1 + e0);
            const uint2 q2 = *reinterpret_cast<const uint2*>(p.st2 + e0);
            float gr[8];
            load8(p.grad, p.grad_dtype, e0, gr);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float c1 = u2f(((k < 4 ? q1.x : q1.y) >> (8 * (k & 3))) & 0xffu);
                const float c2 = u2f(((k < 4 ? q2.x : q2.y) >> (8 * (k & 3))) & 0xffu);
                float m = rb<BF>(__fsub_rn(t1, __fmul_rn(c1, s1)));
                const float r2 = __fsub_rn(t2, __fmul_rn(c2, s2));
                float d = rb<BF>(__fmul_rn(r2, r2));
                adam_moments<BF>(p.h, gr[k], m, d);
                t = __fadd_rn(t, rb<BF>(__fdiv_rn(fabsf(m), d)));
            }
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
        if (active && (threadIdx.x & 15) == 0) stat_out[w >> 4] = t;
    }
}

// ---- many small dense bf16 tensors ---------------------------------------------------------------
__global__ void __launch_bounds__(256) k_adam_dense_multi(const lq_dense_slot* __restrict__ table, const lq_adam_hyper h) {
    const lq_dense_slot t = table[blockIdx.y];
    __nv_bfloat16* pw = reinterpret_cast<__nv_bfloat16*>(t.param);
    const __nv_bfloat16* pg = reinterpret_cast<const __nv_bfloat16*>(t.grad);
    __nv_bfloat16* p1 = reinterpret_cast<__nv_bfloat16*>(t.state1);
    __nv_bfloat16* p2 = reinterpret_cast<__nv_bfloat16*>(t.state2);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < t.numel; i += (int64_t)gridDim.x * blockDim.x) {
        float m = __bfloat162float(p1[i]);
        const float s2 = __bfloat162float(p2[i]);
        float d = rb<true>(__fmul_rn(s2, s2));                             // state2 * state2 (utils/quant.py:1092)
        adam_moments<true>(h, __bfloat162float(pg[i]), m, d);
        const float w = adam_apply<true>(h, __bfloat162float(pw[i]), m, d);
        p1[i] = __float2bfloat16_rn(m);
        p2[i] = __float2bfloat16_rn(d);
        pw[i] = __float2bfloat16_rn(w);
    }
}

// ---- 8-bit stochastic gradient accumulator: GradientQTensor (utils/quant.py:846-921) ----------------------------
// One CTA per weight row.  FIRST (set_value): scale = clamp(4 * absmax(row), 1e-5) / 127 in the gradient's dtype, then
// q = clamp(round_half_even(f / scale + noise), -128, 127).  Otherwise (add_): f <- q * scale + f first, scale kept.
// noise: explicit fp32 buffer, or the library's Philox stream (one block per 8 elements), rounded to the chain dtype
// like the reference's noise tensor.
template <bool BF, bool FIRST, int DITHER>
__global__ void __launch_bounds__(256) k_gradq(const void* __restrict__ f, int dtype, int cols, int8_t* __restrict__ q,
                                               void* __restrict__ scale, const float* __restrict__ noise, uint64_t seed,
                                               uint64_t stream_id) {
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    const int words = cols >> 3;
    float s;
    if (FIRST) {
        float am = 0.0f;
        for (int w = threadIdx.x; w < words; w += 256) {
            float v[8];
            load8(f, dtype, row * cols + (int64_t)w * 8, v);
#pragma unroll
            for (int k = 0; k < 8; ++k) am = fmaxf(am, fabsf(v[k]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) am = fmaxf(am, red[i]);
        const float vmax = rb<BF>(__fmul_rn(am, 4.0f));
        s = rb<BF>(__fdiv_rn(fmaxf(vmax, rb<BF>(1e-5f)), 127.0f));
        if (threadIdx.x == 0) {
            if (dtype == LQ_BF16) reinterpret_cast<__nv_bfloat16*>(scale)[row] = __float2bfloat16_rn(s);
            else reinterpret_cast<float*>(scale)[row] = s;
        }
    } else {
        s = load1(scale, dtype, row);
    }
    for (int w = threadIdx.x; w < words; w += 256) {
        const int64_t e0 = row * cols + (int64_t)w * 8;
        float v[8], u[8];
        load8(f, dtype, e0, v);
        if (DITHER == LQ_DITHER_EXPLICIT) load8(noise, LQ_F32, e0, u);
        else philox_dither8(seed, stream_id, (uint64_t)(e0 >> 3), u);
        uint2 old = make_uint2(0u, 0u);
        if (!FIRST) old = *reinterpret_cast<const uint2*>(q + e0);
        uint32_t b[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float x = v[k];
            if (!FIRST) {
                const uint32_t byte = ((k < 4 ? old.x : old.y) >> (8 * (k & 3))) & 0xffu;
                const float c = __fsub_rn(u2f(byte ^ 0x80u), 128.0f);                 // signed byte
                x = rb<BF>(__fadd_rn(rb<BF>(__fmul_rn(c, s)), x));                    // dequant() + fdata
            }
            float t = rb<BF>(__fadd_rn(rb<BF>(__fdiv_rn(x, s)), rb<BF>(u[k])));
            t = fminf(fmaxf(rne(t), -128.0f), 127.0f);
            b[k] = f2bits(t) & 0xffu;
        }
        *reinterpret_cast<uint2*>(q + e0) = make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24),
                                                      b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24));
    }
}
// get_value(): qdata.to(dtype) * scale
__global__ void __launch_bounds__(256) k_gradq_dequant(const int8_t* __restrict__ q, const void* __restrict__ scale, int dtype,
                                                       int cols, int64_t n_words, void* __restrict__ out) {
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_words; w += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e0 = w * 8;
        const float s = load1(scale, dtype, e0 / cols);
        const uint2 pk = *reinterpret_cast<const uint2*>(q + e0);
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t byte = ((k < 4 ? pk.x : pk.y) >> (8 * (k & 3))) & 0xffu;
            v[k] = __fmul_rn(__fsub_rn(u2f(byte ^ 0x80u), 128.0f), s);                // store8 rounds to the dtype
        }
        store8(out, dtype, e0, v);
    }
}

}  // namespace lq

using namespace lq;

extern "C" {

int lq_adam_a16w4_step(int8_t* codes, int32_t* words, const void* grad, int grad_dtype, const void* scales,
                       const void* zeros, int qp_dtype, int64_t numel, int group, uint8_t* state1, float* scale1,
                       float* tmax1, uint8_t* state2, float* scale2, float* tmax2, int opt_block,
                       const lq_adam_hyper* hyper, const lq_requant_opts* opts, lq_stream_t stream) {
    if (numel == 0) return LQ_OK;
    AdamParams p{};
    int rc = fill_requant(p.rq, opts, numel, group);
    if (rc) return rc;
    if (!hyper || !codes || !words || !grad || !scales || !zeros || !state1 || !scale1 || !tmax1 || !state2 || !scale2 ||
        !tmax2 || !dtype_ok(grad_dtype) || !dtype_ok(qp_dtype) || !aligned(codes, 4) || !aligned(words, 4) ||
        !aligned(grad, 16) || !aligned(state1, 8) || !aligned(state2, 8))
        return LQ_EINVAL;
    if ((opt_block != 2048 && opt_block != 128) || numel % opt_block != 0) return LQ_EINVAL;
    // the chain dtype is the gradient's; mixed gradient / qparam dtypes promote differently op by op in torch
    if (grad_dtype != qp_dtype || opts->math_dtype != grad_dtype) return LQ_EUNSUPPORTED;
    if ((rc = ensure_device_for(codes)) != LQ_OK) return rc;
    p.rq.codes_in = codes; p.rq.words_in = words; p.rq.codes_out = codes; p.rq.words_out = words;
    p.rq.scales = scales; p.rq.zeros = zeros; p.rq.qp_dtype = qp_dtype;
    p.grad = grad; p.grad_dtype = grad_dtype;
    p.st1 = state1; p.sc1 = scale1; p.tm1 = tmax1; p.st2 = state2; p.sc2 = scale2; p.tm2 = tmax2;
    p.opt_shift = opt_block == 2048 ? 11 : 7;
    p.n_tiles = (p.rq.n_words + 255) / 256;
    p.h = *hyper;
    const bool bf = grad_dtype == LQ_BF16;
    cudaStream_t st = LQ_ST(stream);
    if (opts->codec == LQ_CODEC_THREEFOLD && opts->dither == LQ_DITHER_HASH) {
        if (bf && p.rq.group_shift >= 3 && p.rq.n_words < ((int64_t)1 << 31) && opts->mu_enc >= 0 && opts->mu_enc <= 3 &&
            opts->mu_dec >= 0 && opts->mu_dec <= 3 && !getenv("LQ_REQUANT_GENERIC")) {
            rc = ensure_encz_table(opts->mu_enc, opts->v0, st);
            if (rc) return rc;
            static bool attr_done[64][2] = {};
            int dev = 0;
            cudaGetDevice(&dev);
            const int ur = p.rq.has_residual ? 1 : 0;
            if (dev >= 0 && dev < 64 && !attr_done[dev][ur]) {
                cudaError_t e = ur ? cudaFuncSetAttribute(k_adam_a16w4_fast<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ADAM_FAST_SMEM)
                                   : cudaFuncSetAttribute(k_adam_a16w4_fast<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ADAM_FAST_SMEM);
                if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(k_adam_a16w4_fast)"); return LQ_ECUDA; }
                attr_done[dev][ur] = true;
            }
            const int64_t cap = (int64_t)sm_count() * 3;
            const int grid = (int)(p.n_tiles < cap ? p.n_tiles : cap);
            if (ur) k_adam_a16w4_fast<true><<<grid, 256, ADAM_FAST_SMEM, st>>>(p, opts->mu_enc);
            else k_adam_a16w4_fast<false><<<grid, 256, ADAM_FAST_SMEM, st>>>(p, opts->mu_enc);
            return check_launch("k_adam_a16w4_fast");
        }
        return launch_adam<4, LQ_CODEC_THREEFOLD, LQ_DITHER_HASH>(p, bf, st);
    }
    if (opts->codec == LQ_CODEC_THREEFOLD && opts->dither == LQ_DITHER_PHILOX) return launch_adam<4, LQ_CODEC_THREEFOLD, LQ_DITHER_PHILOX>(p, bf, st);
    if (opts->codec == LQ_CODEC_UNIFORM16 && opts->dither == LQ_DITHER_PHILOX) return launch_adam<4, LQ_CODEC_UNIFORM16, LQ_DITHER_PHILOX>(p, bf, st);
    return LQ_EUNSUPPORTED;
}

int lq_adam_a8w8_step(int8_t* codes, int32_t* words, const void* grad, int grad_dtype, const void* qscales, int qp_dtype,
                      int64_t rows, int64_t cols, uint8_t* state1, float* scale1, float* tmax1, uint8_t* state2, float* scale2,
                      float* tmax2, int opt_block, const lq_adam_hyper* hyper, const lq_requant_opts* opts, lq_stream_t stream) {
    if (rows == 0 || cols == 0) return LQ_OK;
    if (rows < 0 || cols < 0) return LQ_EINVAL;
    AdamParams p{};
    const int64_t numel = rows * cols;
    int rc = fill_requant(p.rq, opts, numel, cols);          // one scale per weight row: the "group" is the row
    if (rc) return rc;
    if (!hyper || !codes || !words || !grad || !qscales || !state1 || !scale1 || !tmax1 || !state2 || !scale2 || !tmax2 ||
        !dtype_ok(grad_dtype) || !dtype_ok(qp_dtype) || !aligned(codes, 8) || !aligned(words, 4) || !aligned(grad, 16) ||
        !aligned(state1, 8) || !aligned(state2, 8))
        return LQ_EINVAL;
    if ((opt_block != 2048 && opt_block != 128) || numel % opt_block != 0) return LQ_EINVAL;
    if (grad_dtype != qp_dtype || opts->math_dtype != grad_dtype) return LQ_EUNSUPPORTED;
    if ((rc = ensure_device_for(codes)) != LQ_OK) return rc;
    p.rq.codes_in = codes; p.rq.words_in = words; p.rq.codes_out = codes; p.rq.words_out = words;
    p.rq.scales = qscales; p.rq.zeros = nullptr; p.rq.qp_dtype = qp_dtype;
    p.grad = grad; p.grad_dtype = grad_dtype;
    p.st1 = state1; p.sc1 = scale1; p.tm1 = tmax1; p.st2 = state2; p.sc2 = scale2; p.tm2 = tmax2;
    p.opt_shift = opt_block == 2048 ? 11 : 7;
    p.n_tiles = (p.rq.n_words + 255) / 256;
    p.h = *hyper;
    const bool bf = grad_dtype == LQ_BF16;
    cudaStream_t st = LQ_ST(stream);
    if (opts->codec == LQ_CODEC_THREEFOLD && opts->dither == LQ_DITHER_HASH) return launch_adam<8, LQ_CODEC_THREEFOLD, LQ_DITHER_HASH>(p, bf, st);
    if (opts->codec == LQ_CODEC_THREEFOLD && opts->dither == LQ_DITHER_PHILOX) return launch_adam<8, LQ_CODEC_THREEFOLD, LQ_DITHER_PHILOX>(p, bf, st);
    return LQ_EUNSUPPORTED;
}

int lq_adam_moment_stat(const void* grad, int grad_dtype, int64_t numel, const uint8_t* state1, const float* scale1,
                        const float* tmax1, const uint8_t* state2, const float* scale2, const float* tmax2, int opt_block,
                        const lq_adam_hyper* hyper, float* stat_out, lq_stream_t stream) {
    if (numel == 0) return LQ_OK;
    if (!grad || !state1 || !scale1 || !tmax1 || !state2 || !scale2 || !tmax2 || !hyper || !stat_out || !dtype_ok(grad_dtype) ||
        numel < 0 || (numel % 128) != 0 || !aligned(grad, 16) || !aligned(state1, 8) || !aligned(state2, 8))
        return LQ_EINVAL;
    if ((opt_block != 2048 && opt_block != 128) || numel % opt_block != 0) return LQ_EINVAL;
    int rc = ensure_device_for(grad);
    if (rc != LQ_OK) return rc;
    AdamParams p{};
    p.rq.n_words = numel / 8;
    p.grad = grad; p.grad_dtype = grad_dtype;
    p.st1 = const_cast<uint8_t*>(state1); p.sc1 = const_cast<float*>(scale1); p.tm1 = const_cast<float*>(tmax1);
    p.st2 = const_cast<uint8_t*>(state2); p.sc2 = const_cast<float*>(scale2); p.tm2 = const_cast<float*>(tmax2);
    p.opt_shift = opt_block == 2048 ? 11 : 7;
    p.n_tiles = (p.rq.n_words + 255) / 256;
    p.h = *hyper;
    const int grid = grid_for(p.rq.n_words, 256, 8);
    if (grad_dtype == LQ_BF16) k_adam_moment_stat<true><<<grid, 256, 0, LQ_ST(stream)>>>(p, stat_out);
    else k_adam_moment_stat<false><<<grid, 256, 0, LQ_ST(stream)>>>(p, stat_out);
    return check_launch("k_adam_moment_stat");
}

int lq_gradq_accumulate(const void* fdata, int dtype, int64_t rows, int64_t cols, int8_t* qdata, void* scale, int first,
                        const lq_requant_opts* opts, lq_stream_t stream) {
    if (rows == 0 || cols == 0) return LQ_OK;
    if (!fdata || !qdata || !scale || !opts || !dtype_ok(dtype) || rows < 0 || cols < 0 || (cols % 8) != 0 || cols >= (1ll << 31) ||
        rows >= (1ll << 31) || !aligned(fdata, 16) || !aligned(qdata, 8))
        return LQ_EINVAL;
    if (opts->dither == LQ_DITHER_EXPLICIT && (!opts->dither_buf || !aligned(opts->dither_buf, 16))) return LQ_EINVAL;
    if (opts->dither != LQ_DITHER_EXPLICIT && opts->dither != LQ_DITHER_PHILOX) return LQ_EUNSUPPORTED;
    int rc = ensure_device_for(fdata);
    if (rc != LQ_OK) return rc;
    const bool bf = dtype == LQ_BF16, ex = opts->dither == LQ_DITHER_EXPLICIT;
    cudaStream_t st = LQ_ST(stream);
#define LQ_GRADQ(BFv, FIRSTv, DITHv) k_gradq<BFv, FIRSTv, DITHv><<<(unsigned)rows, 256, 0, st>>>(fdata, dtype, (int)cols, qdata, scale, opts->dither_buf, opts->seed, opts->stream_id)
    if (bf) { if (first) { if (ex) LQ_GRADQ(true, true, LQ_DITHER_EXPLICIT); else LQ_GRADQ(true, true, LQ_DITHER_PHILOX); }
              else { if (ex) LQ_GRADQ(true, false, LQ_DITHER_EXPLICIT); else LQ_GRADQ(true, false, LQ_DITHER_PHILOX); } }
    else { if (first) { if (ex) LQ_GRADQ(false, true, LQ_DITHER_EXPLICIT); else LQ_GRADQ(false, true, LQ_DITHER_PHILOX); }
           else { if (ex) LQ_GRADQ(false, false, LQ_DITHER_EXPLICIT); else LQ_GRADQ(false, false, LQ_DITHER_PHILOX); } }
#undef LQ_GRADQ
    return check_launch("k_gradq");
}

int lq_gradq_dequant(const int8_t* qdata, const void* scale, int dtype, int64_t rows, int64_t cols, void* out, lq_stream_t stream) {
    if (rows == 0 || cols == 0) return LQ_OK;
    if (!qdata || !scale || !out || !dtype_ok(dtype) || rows < 0 || cols < 0 || (cols % 8) != 0 || cols >= (1ll << 31) ||
        !aligned(qdata, 8) || !aligned(out, 16))
        return LQ_EINVAL;
    int rc = ensure_device_for(qdata);
    if (rc != LQ_OK) return rc;
    const int64_t n_words = rows * cols / 8;
    k_gradq_dequant<<<grid_for(n_words, 256, 8), 256, 0, LQ_ST(stream)>>>(qdata, scale, dtype, (int)cols, n_words, out);
    return check_launch("k_gradq_dequant");
}

int lq_adam_dense_multi(const lq_dense_slot* table, int n_tensors, int64_t max_numel, const lq_adam_hyper* hyper,
                        lq_stream_t stream) {
    if (n_tensors == 0 || max_numel == 0) return LQ_OK;
    if (!table || !hyper || n_tensors < 0 || n_tensors > 65535 || max_numel < 0) return LQ_EINVAL;
    int rc = ensure_device_for(table);
    if (rc != LQ_OK) return rc;
    int64_t bx = (max_numel + 255) / 256;
    if (bx > 64) bx = 64;
    dim3 grid((unsigned)bx, (unsigned)n_tensors);
    k_adam_dense_multi<<<grid, 256, 0, LQ_ST(stream)>>>(table, *hyper);
    return check_launch("k_adam_dense_multi");
}

}  // extern "C"
