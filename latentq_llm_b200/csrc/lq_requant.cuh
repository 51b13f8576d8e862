// Device-side building blocks of the latent-weight requantize, shared by the streaming kernels and the fused
// optimizer step: dtype-generic 8-element loads/stores, conversion-free rounding helpers, and the two halves
// of the per-word chain (reconstruct the latent weights / quantize them back to codes + residual nibbles).
#pragma once
#include <mutex>

#include "lq_common.cuh"

namespace lq {

// ---- 8-element vector load / store in the tensor's dtype -------------------------------------
__device__ __forceinline__ void load8(const void* base, int dtype, int64_t e0, float (&v)[8]) {
    if (dtype == LQ_BF16) {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + e0));
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + e0);
        float4 a = __ldg(p), b = __ldg(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}
__device__ __forceinline__ void store8(void* base, int dtype, int64_t e0, const float (&v)[8]) {
    if (dtype == LQ_BF16) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = f32_to_bf16_bits(v[2 * i]) | (f32_to_bf16_bits(v[2 * i + 1]) << 16);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + e0) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + e0);
        p[0] = make_float4(v[0], v[1], v[2], v[3]);
        p[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}
__device__ __forceinline__ float load1(const void* base, int dtype, int64_t i) {
    return dtype == LQ_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i])
                            : __ldg(reinterpret_cast<const float*>(base) + i);
}

// =================================================================================================
// Latent-weight requantize
// =================================================================================================
struct RequantParams {
    const void* w_in; int w_dtype;
    const void* codes_in; const int32_t* words_in;
    const void* delta; int delta_dtype;
    const void* scales; const void* zeros; int qp_dtype;
    int64_t n_words; int64_t group; int group_shift;
    void* codes_out; int32_t* words_out;
    Curve enc, dec;
    float v0; uint64_t seed, stream_id; const float* dither_buf;
    int has_residual, res_round_bf16;
};

// ---- conversion-free arithmetic helpers -------------------------------------------------------
// int<->float conversions, rintf and roundf issue on the slow conversion pipe; the chain below uses
// magic-number adds instead (exact for the value ranges stated).
constexpr float MAGIC_RNE = 12582912.0f;            // 1.5 * 2^23
// small non-negative integer (< 2^22) -> float, exactly
__device__ __forceinline__ float u2f(uint32_t n) { return __fsub_rn(__uint_as_float(0x4B000000u | n), 8388608.0f); }
// round-half-even of x for |x| < 2^22 (falls back to rintf beyond)
__device__ __forceinline__ float rne(float x) {
    if (fabsf(x) < 4194304.0f) return __fsub_rn(__fadd_rn(x, MAGIC_RNE), MAGIC_RNE);
    return rintf(x);
}
// integer-valued float in [-2^21, 2^21] -> its two's-complement low bits
__device__ __forceinline__ uint32_t f2bits(float q) { return __float_as_uint(__fadd_rn(q, MAGIC_RNE)); }
// round-half-away of y for |y| < 2^22: half-even first, then push ties that went towards zero
__device__ __forceinline__ float rha(float y) {
    float q = __fsub_rn(__fadd_rn(y, MAGIC_RNE), MAGIC_RNE);
    float d = __fsub_rn(y, q);
    if (fabsf(d) == 0.5f && (d > 0.0f) == (y > 0.0f)) q = __fadd_rn(q, copysignf(1.0f, y));
    return q;
}
// |x|*499 + v0 minus its round-half-away integer part (.cu:49-51), v >= 0 assumed small
__device__ __forceinline__ float hash_dither_fast(float x, float v0) {
    float v = __fmaf_rn(fabsf(x), 499.0f, v0);
    return __fsub_rn(v, rha(v));
}
__device__ __forceinline__ uint32_t res3_encode_fast(float x, float v, const Curve& c, float& carry) {
    float S = fabsf(x), q;
    if (S < c.b1) {
        q = rha(__fmaf_rn(x, c.c1, v));
    } else {
        const bool mid = S < c.b2;
        float r = __fadd_rn(rha(__fmaf_rn(__fsub_rn(S, mid ? c.b1 : c.b2), mid ? c.c2 : c.c3, v)), mid ? c.t1 : c.t2);
        q = (x < 0.0f) ? -r : r;
    }
    if (q > 7.5f) { carry = 1.0f; return 1u; }
    carry = 0.0f;
    float t = q + 8.0f;
    return (t <= 0.0f) ? 0u : (f2bits(t) & 15u);
}
__device__ __forceinline__ float res3_decode_fast(uint32_t nib, const Curve& c) {
    float s = __fsub_rn(u2f(nib), 8.0f);
    if (s < -c.t2) return __fmaf_rn(s + c.t2, c.ic3, -c.b2);
    if (s < -c.t1) return __fmaf_rn(s + c.t1, c.ic2, -c.b1);
    if (s <= c.t1) return __fmul_rn(s, c.ic1);
    if (s <= c.t2) return __fmaf_rn(s - c.t1, c.ic2, c.b1);
    return __fmaf_rn(s - c.t2, c.ic3, c.b2);
}
// bf16 rounding (half-even) in integer arithmetic; finite inputs
template <bool BF> __device__ __forceinline__ float rb(float x) {
    if (!BF) return x;
    uint32_t u = __float_as_uint(x);
    u += 0x7fffu + ((u >> 16) & 1u);
    return __uint_as_float(u & 0xffff0000u);
}
// correctly rounded a/s from r = RN(1/s); only large |a| needs the slow path (tiny |a| cannot change any
// output of the chain: the quotient stays below 2^-19 either way)
__device__ __forceinline__ float div_fast(float a, float s, float r, bool scale_ok) {
    if (scale_ok && fabsf(a) <= 1.1529215e18f) {
        float q = __fmul_rn(a, r);
        float e = __fmaf_rn(-q, s, a);
        q = __fmaf_rn(e, r, q);
        e = __fmaf_rn(-q, s, a);
        return __fmaf_rn(e, r, q);
    }
    return __fdiv_rn(a, s);
}

// WBITS 4: codes are nibble pairs (4 bytes per 8 elements), zero point per group, clamp [0,15].
// WBITS 8: codes are int8 (8 bytes per 8 elements), no zero point, clamp [-128,127].
// Reconstruct the 8 latent weights of word w: either the dense input, or codes dequantized + decoded residual
// (+ the optional update), every step rounded as the reference's tensor ops round it.
template <int WBITS, int CODEC, bool BF>
__device__ __forceinline__ void latent_load(const RequantParams& p, const int64_t w, const float s, const float z,
                                            float (&lat)[8]) {
        const int64_t e0 = w * 8;
        if (p.w_in) {
            load8(p.w_in, p.w_dtype, e0, lat);
        } else {
            // issue every load of this word first
            uint32_t pk0 = 0, pk1 = 0, rw = 0;
            if (WBITS == 4) pk0 = __ldg(reinterpret_cast<const uint32_t*>(p.codes_in) + w);
            else { uint2 t = __ldg(reinterpret_cast<const uint2*>(p.codes_in) + w); pk0 = t.x; pk1 = t.y; }
            const bool use_res = (CODEC != LQ_CODEC_NONE) && p.has_residual;
            if (use_res) rw = (uint32_t)__ldg(p.words_in + w);
            float d[8];
            if (p.delta) load8(p.delta, p.delta_dtype, e0, d);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float c;
                if (WBITS == 4) c = u2f((pk0 >> (8 * (k >> 1) + ((k & 1) ? 0 : 4))) & 15u);
                else {   // signed byte: (b ^ 0x80) - 128
                    uint32_t b = ((k < 4 ? pk0 : pk1) >> (8 * (k & 3))) & 0xffu;
                    c = __fsub_rn(u2f(b ^ 0x80u), 128.0f);
                }
                lat[k] = rb<BF>(__fmul_rn(rb<BF>(__fsub_rn(c, z)), s));
            }
            if (use_res) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    uint32_t nib = (rw >> (28 - 4 * k)) & 15u;
                    float rv = (CODEC == LQ_CODEC_UNIFORM16) ? __fmaf_rn(u2f(nib), 0.0625f, -0.5f) : rb<true>(res3_decode_fast(nib, p.dec));
                    lat[k] = rb<BF>(__fadd_rn(rb<BF>(__fmul_rn(rv, s)), lat[k]));
                }
            }
            if (p.delta) {
#pragma unroll
                for (int k = 0; k < 8; ++k) lat[k] = rb<BF>(__fadd_rn(lat[k], d[k]));
            }
        }
}

// What the chain computes from Z = w/scale + zero alone (A16W4, 3-fold codec, hash dither, bf16 chain):
// round-half-even, residual, its 4-bit code and carry, clamp.  Returns code << 4 | residual nibble.  Same operations,
// in the same order, as latent_store below performs for that configuration (it is what the fast path tabulates).
__device__ __forceinline__ uint32_t encode_from_z_w4_hash_bf16(float Z, const Curve& enc, float v0) {
    float qf = rne(Z);
    const float r = rb<true>(__fsub_rn(Z, qf));
    float carry = 0.0f;
    const uint32_t nib = res3_encode_fast(r, hash_dither_fast(r, v0), enc, carry) & 15u;
    qf = rb<true>(__fadd_rn(qf, carry));
    qf = fminf(fmaxf(qf, 0.0f), 15.0f);
    return ((f2bits(qf) & 15u) << 4) | nib;
}
// int8 codes (A8W8: no zero point, clamp [-128, 127]); returns (code & 0xff) | nibble << 8
__device__ __forceinline__ uint32_t encode_from_z_w8_hash_bf16(float Z, const Curve& enc, float v0) {
    float qf = rne(Z);
    const float r = rb<true>(__fsub_rn(Z, qf));
    float carry = 0.0f;
    const uint32_t nib = res3_encode_fast(r, hash_dither_fast(r, v0), enc, carry) & 15u;
    qf = rb<true>(__fadd_rn(qf, carry));
    qf = fminf(fmaxf(qf, -128.0f), 127.0f);
    return (f2bits(qf) & 0xffu) | (nib << 8);
}
// Same with an external dither value v in [-0.5, 0.5) (explicit buffer or Philox) instead of the hash of the residual.
__device__ __forceinline__ uint32_t encode_from_z_w4_dither_bf16(float Z, float v, const Curve& enc) {
    float qf = rne(Z);
    const float r = rb<true>(__fsub_rn(Z, qf));
    float carry = 0.0f;
    const uint32_t nib = res3_encode_fast(r, v, enc, carry) & 15u;
    qf = rb<true>(__fadd_rn(qf, carry));
    qf = fminf(fmaxf(qf, 0.0f), 15.0f);
    return ((f2bits(qf) & 15u) << 4) | nib;
}

// Quantize 8 latent weights to codes + residual nibbles and store both.
template <int WBITS, int CODEC, int DITHER, bool BF>
__device__ __forceinline__ void latent_store(const RequantParams& p, const int64_t w, const float s, const float z,
                                             const float (&lat)[8]) {
        const int64_t e0 = w * 8;
        const float rs = __frcp_rn(s);
        const bool s_ok = fastdiv_ok_scale(s);
        float u[8];
        if (CODEC != LQ_CODEC_NONE) {
            if (DITHER == LQ_DITHER_EXPLICIT) load8(p.dither_buf, LQ_F32, e0, u);
            else if (DITHER == LQ_DITHER_PHILOX) philox_dither8(p.seed, p.stream_id, (uint64_t)w, u);
        }

        uint32_t rword = 0, q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float Z = rb<BF>(div_fast(lat[k], s, rs, s_ok));
            if (WBITS == 4) Z = rb<BF>(__fadd_rn(Z, z));
            float qf = rne(Z);
            float r = rb<BF>(__fsub_rn(Z, qf));
            float carry = 0.0f;
            uint32_t nib = 0;
            if (CODEC != LQ_CODEC_NONE) {
                if (p.res_round_bf16) r = rb<true>(r);
                if (CODEC == LQ_CODEC_UNIFORM16) {
                    // (r+0.5)*16 == fma(r,16,8) exactly (scaling by 16 commutes with rounding); then + dither, round-half-even
                    uint32_t n = f2bits(__fadd_rn(__fmaf_rn(r, 16.0f, 8.0f), u[k])) & 31u;
                    if (n >= 16u) { carry = 1.0f; nib = 0u; } else nib = n;
                } else {
                    float v = (DITHER == LQ_DITHER_HASH) ? hash_dither_fast(r, p.v0) : u[k];
                    nib = res3_encode_fast(r, v, p.enc, carry) & 15u;
                }
            }
            qf = rb<BF>(__fadd_rn(qf, carry));
            qf = (WBITS == 4) ? fminf(fmaxf(qf, 0.0f), 15.0f) : fminf(fmaxf(qf, -128.0f), 127.0f);
            q[k] = f2bits(qf) & 0xffu;
            rword = (rword << 4) | nib;
        }
        if (CODEC != LQ_CODEC_NONE) p.words_out[w] = (int32_t)rword;
        if (WBITS == 4) {
            uint32_t pk = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) pk |= (((q[2 * k] & 15u) << 4) | (q[2 * k + 1] & 15u)) << (8 * k);
            reinterpret_cast<uint32_t*>(p.codes_out)[w] = pk;
        } else {
            uint2 pk;
            pk.x = q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24);
            pk.y = q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24);
            reinterpret_cast<uint2*>(p.codes_out)[w] = pk;
        }
}

template <int WBITS, int CODEC, int DITHER, bool BF>
__device__ __forceinline__ void requant_word(const RequantParams& p, const int64_t w) {
    const int64_t e0 = w * 8;
    const int64_t g = p.group_shift >= 0 ? (e0 >> p.group_shift) : (e0 / p.group);
    const float s = load1(p.scales, p.qp_dtype, g);
    const float z = (WBITS == 4) ? load1(p.zeros, p.qp_dtype, g) : 0.0f;
    float lat[8];
    latent_load<WBITS, CODEC, BF>(p, w, s, z, lat);
    latent_store<WBITS, CODEC, DITHER, BF>(p, w, s, z, lat);
}


// ---- host-side helpers shared by the entry points ----------------------------------------------
#define LQ_ST(s) reinterpret_cast<cudaStream_t>(s)
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static inline int grid_for(int64_t work_items, int threads, int ctas_per_sm) {
    int64_t want = (work_items + threads - 1) / threads;
    int64_t cap = (int64_t)sm_count() * ctas_per_sm;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

static inline int fill_requant(RequantParams& p, const lq_requant_opts* o, int64_t numel, int64_t group) {
    if (!o || numel <= 0 || (numel % 8) != 0 || group <= 0 || (group % 8) != 0 || (numel % group) != 0) return LQ_EINVAL;
    if (o->math_dtype != LQ_F32 && o->math_dtype != LQ_BF16) return LQ_EINVAL;
    if (o->codec != LQ_CODEC_NONE && o->dither == LQ_DITHER_EXPLICIT && (!o->dither_buf || !aligned(o->dither_buf, 16))) return LQ_EINVAL;
    p.n_words = numel / 8; p.group = group; p.group_shift = -1;
    if ((group & (group - 1)) == 0) { int sh = 0; while (((int64_t)1 << sh) < group) ++sh; p.group_shift = sh; }
    p.enc = curve_for_level(o->mu_enc); p.dec = curve_for_level(o->mu_dec);
    p.v0 = o->v0; p.seed = o->seed; p.stream_id = o->stream_id; p.dither_buf = o->dither_buf;
    p.has_residual = o->has_residual; p.res_round_bf16 = o->res_round_bf16;
    return LQ_OK;
}
static inline bool dtype_ok(int d) { return d == LQ_F32 || d == LQ_BF16; }


// ---- table of the bf16 fast paths: everything after Z as one byte (each translation unit that launches a kernel
// reading it holds its own copy; built once per device, curve level and hash offset) ---------------------------
constexpr int ENCZ_TABLE_ENTRIES = 65536;               // every bf16 pattern of Z = w/scale + zero
static __device__ uint8_t g_encz_table[4][ENCZ_TABLE_ENTRIES]; // one per curve level; entry = final code << 4 | residual nibble
static __global__ void __launch_bounds__(256) k_build_encz_table(int slot, Curve c, float v0) {
    for (int h = blockIdx.x * blockDim.x + threadIdx.x; h < ENCZ_TABLE_ENTRIES; h += gridDim.x * blockDim.x) {
        const float Z = __uint_as_float((uint32_t)h << 16);
        uint8_t e = 0;                                  // |Z| >= 64, inf, NaN: never looked up (the word takes the generic chain)
        if (fabsf(Z) < 64.0f) e = (uint8_t)encode_from_z_w4_hash_bf16(Z, c, v0);
        g_encz_table[slot][h] = e;
    }
}

static std::mutex g_encz_mutex;
// Builds (once per device, curve level and v0) the encode table the fast path reads.
static inline int ensure_encz_table(int mu, float v0, cudaStream_t st) {
    static bool built[64][4] = {};
    static float built_v0[64][4] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LQ_EUNSUPPORTED;
    const int slot = (mu < 0 || mu > 3) ? 0 : mu;
    std::lock_guard<std::mutex> lock(g_encz_mutex);
    if (built[dev][slot] && built_v0[dev][slot] == v0) return LQ_OK;
    k_build_encz_table<<<128, 256, 0, st>>>(slot, curve_for_level(slot), v0);
    int rc = check_launch("k_build_encz_table");
    if (rc) return rc;
    // first use only: make the table visible to every stream before anyone else may read it
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { set_cuda_error(e, "cudaStreamSynchronize"); return LQ_ECUDA; }
    built[dev][slot] = true; built_v0[dev][slot] = v0;
    return LQ_OK;
}


}  // namespace lq
