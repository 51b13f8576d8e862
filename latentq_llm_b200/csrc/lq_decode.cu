// Decode-side operations around the quantized GEMMs of a Llama-architecture layer (bf16, sm_100a): what the
// reference fuses around its int4 matmul in PTQ/quant —
//   * RMSNorm                      (PTQ/quant/triton_norm.py:7-39), here with the residual add that precedes it,
//   * rotate-half RoPE on q and k  (PTQ/quant/fused_attn.py:8-58), here writing k and v straight into the KV cache,
//   * silu(gate) * up              (epilogue of PTQ/quant/fused_mlp.py:84-168),
//   * single-query attention over the KV cache (the reference calls F.scaled_dot_product_attention,
//     PTQ/quant/fused_attn.py:148-149).
// A decode step then is nine launches per layer instead of the ~45 elementwise kernels of the eager modules.
// All kernels are HBM/L2 streaming kernels over a few hundred KB: one pass, 16-byte accesses, no scratch
// besides the attention's split partials.
//
// Rounding: `hf_rounding != 0` reproduces the bf16 tensor-op chain of the eager HF modules (every op result
// rounded to bf16); 0 keeps fp32 up to the single final cast like the reference's Triton kernels do.
#include "lq_common.cuh"

namespace lq {

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// h += delta (optional); y = RMSNorm(h) * gamma.  One CTA per token row.
// ---------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
__global__ void __launch_bounds__(NORM_THREADS) k_add_rmsnorm(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                                                               const __nv_bfloat16* __restrict__ gamma, float eps,
                                                               __nv_bfloat16* __restrict__ y, int K, int hf_rounding) {
    __shared__ float red[NORM_THREADS / 32];
    pdl_launch_dependents();                          // (decode chain) the successor may be launched; it waits for this grid
    pdl_wait();                                       // h / delta may be the predecessor's output
    const size_t row = (size_t)blockIdx.x * K;
    uint4* hv = reinterpret_cast<uint4*>(h + row);
    const uint4* dv = delta ? reinterpret_cast<const uint4*>(delta + row) : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < K / 8; i += NORM_THREADS) {
        uint4 a = hv[i];
        uint32_t w[4] = {a.x, a.y, a.z, a.w};
        if (dv) {                                      // residual + hidden_states: one bf16 rounding of the fp32 sum
            const uint4 d = __ldg(dv + i);
            const uint32_t e[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = pack_bf2(__fadd_rn(bf_lo(w[j]), bf_lo(e[j])), __fadd_rn(bf_hi(w[j]), bf_hi(e[j])));
            hv[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float lo = bf_lo(w[j]), hi = bf_hi(w[j]); ss = fmaf(lo, lo, ss); ss = fmaf(hi, hi, ss); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int wv = 0; wv < NORM_THREADS / 32; ++wv) tot += red[wv];          // same order in every thread
    const float rstd = hf_rounding ? rsqrtf(tot / (float)K + eps) : 1.0f / sqrtf(tot / (float)K + eps);
    const uint4* gv = reinterpret_cast<const uint4*>(gamma);
    uint4* yv = reinterpret_cast<uint4*>(y + row);
    for (int i = threadIdx.x; i < K / 8; i += NORM_THREADS) {
        const uint4 a = hv[i], g = __ldg(gv + i);          // this thread wrote hv[i] itself
        const uint32_t w[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float lo = __fmul_rn(bf_lo(w[j]), rstd), hi = __fmul_rn(bf_hi(w[j]), rstd);
            if (hf_rounding) { lo = bf16r(lo); hi = bf16r(hi); }
            o[j] = pack_bf2(__fmul_rn(lo, bf_lo(gw[j])), __fmul_rn(hi, bf_hi(gw[j])));
        }
        yv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Register-resident variant for K <= 2048 * VPT: every thread requests all its vectors of h, delta and gamma before
// anything is reduced (one round of memory latency instead of three), and the row is never re-read.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS) k_add_rmsnorm_r(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                                                                 const __nv_bfloat16* __restrict__ gamma, float eps,
                                                                 __nv_bfloat16* __restrict__ y, int K, int hf_rounding) {
    __shared__ float red[NORM_THREADS / 32];
    const uint4* gv = reinterpret_cast<const uint4*>(gamma);
    const int nvec = K / 8;
    uint4 g[VPT], a[VPT], d[VPT];
#pragma unroll
    for (int u = 0; u < VPT; ++u) {                   // gamma is a parameter: fetched before the dependency wait
        const int i = threadIdx.x + u * NORM_THREADS;
        g[u] = i < nvec ? __ldg(gv + i) : make_uint4(0, 0, 0, 0);
    }
    pdl_launch_dependents();
    pdl_wait();                                       // h / delta may be the predecessor's output
    const size_t row = (size_t)blockIdx.x * K;
    uint4* hv = reinterpret_cast<uint4*>(h + row);
    const uint4* dv = delta ? reinterpret_cast<const uint4*>(delta + row) : nullptr;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = threadIdx.x + u * NORM_THREADS;
        a[u] = i < nvec ? hv[i] : make_uint4(0, 0, 0, 0);
        d[u] = (dv && i < nvec) ? __ldg(dv + i) : make_uint4(0, 0, 0, 0);
    }
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&a[u]);
        const uint32_t* e = reinterpret_cast<const uint32_t*>(&d[u]);
        if (dv) {
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = pack_bf2(__fadd_rn(bf_lo(w[j]), bf_lo(e[j])), __fadd_rn(bf_hi(w[j]), bf_hi(e[j])));
            const int i = threadIdx.x + u * NORM_THREADS;
            if (i < nvec) hv[i] = a[u];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float lo = bf_lo(w[j]), hi = bf_hi(w[j]); ss = fmaf(lo, lo, ss); ss = fmaf(hi, hi, ss); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int wv = 0; wv < NORM_THREADS / 32; ++wv) tot += red[wv];
    const float rstd = hf_rounding ? rsqrtf(tot / (float)K + eps) : 1.0f / sqrtf(tot / (float)K + eps);
    uint4* yv = reinterpret_cast<uint4*>(y + row);
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int i = threadIdx.x + u * NORM_THREADS;
        if (i >= nvec) continue;
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&a[u]);
        const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g[u]);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float lo = __fmul_rn(bf_lo(w[j]), rstd), hi = __fmul_rn(bf_hi(w[j]), rstd);
            if (hf_rounding) { lo = bf16r(lo); hi = bf16r(hi); }
            o[j] = pack_bf2(__fmul_rn(lo, bf_lo(gw[j])), __fmul_rn(hi, bf_hi(gw[j])));
        }
        yv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---------------------------------------------------------------------------------------------
// RoPE (rotate-half) on the q and k heads of a fused qkv row, k and v stored into the cache at the token's position.
// grid (token, head of q|k|v), hd/2 threads.  Cache layout [batch, kv head, max_len, hd].
// ---------------------------------------------------------------------------------------------
__global__ void k_rope_kv_store(__nv_bfloat16* __restrict__ qkv, const long long* __restrict__ positions,
                                const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ k_cache,
                                __nv_bfloat16* __restrict__ v_cache, int tokens_per_seq, int Hq, int Hkv, int hd, int max_len,
                                int hf_rounding) {
    const int m = blockIdx.x, head = blockIdx.y, i = threadIdx.x, half = hd >> 1;
    pdl_launch_dependents();
    pdl_wait();                                       // qkv is the predecessor's output
    const long long pos = positions[m];
    __nv_bfloat16* src = qkv + (size_t)m * (size_t)(Hq + 2 * Hkv) * hd + (size_t)head * hd;
    const int b = m / tokens_per_seq;
    if (head >= Hq + Hkv) {                                   // v: plain copy into the cache
        if (pos < 0 || pos >= max_len) return;
        __nv_bfloat16* dst = v_cache + (((size_t)b * Hkv + (head - Hq - Hkv)) * max_len + (size_t)pos) * hd;
        reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
        return;
    }
    const float x = __bfloat162float(src[i]), yv = __bfloat162float(src[i + half]);
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    float ox, oy;
    if (hf_rounding) {        // cos / sin cast to bf16, then q*cos + rotate_half(q)*sin as bf16 tensor ops
        c = bf16r(c); s = bf16r(s);
        ox = __fadd_rn(bf16r(__fmul_rn(x, c)), bf16r(__fmul_rn(-yv, s)));
        oy = __fadd_rn(bf16r(__fmul_rn(yv, c)), bf16r(__fmul_rn(x, s)));
    } else {
        ox = __fsub_rn(__fmul_rn(x, c), __fmul_rn(yv, s));
        oy = __fadd_rn(__fmul_rn(x, s), __fmul_rn(yv, c));
    }
    const __nv_bfloat16 bx = __float2bfloat16_rn(ox), by = __float2bfloat16_rn(oy);
    if (head < Hq) { src[i] = bx; src[i + half] = by; return; }                 // q: in place
    if (pos < 0 || pos >= max_len) return;
    __nv_bfloat16* dst = k_cache + (((size_t)b * Hkv + (head - Hq)) * max_len + (size_t)pos) * hd;
    dst[i] = bx; dst[i + half] = by;
}

// ---------------------------------------------------------------------------------------------
// Single-query attention over the cache: out[b, h, :] = softmax(q . K[0..pos] * scale) . V[0..pos].
// grid (batch * q heads, splits); 128 threads = 16 key slots of 8 lanes, a lane holds hd/8 dims (hd = 64 or 128).
// Each split covers a contiguous range of keys and leaves (max, sum, weighted V) in the workspace; the split
// that finishes last for its (batch, head) combines them (a ticket counter; nobody waits for anybody).
// ---------------------------------------------------------------------------------------------
constexpr int ATT_THREADS = 128, ATT_SLOTS = ATT_THREADS / 8;
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) k_decode_attn(const __nv_bfloat16* __restrict__ q, int q_row_stride,
                                                              const __nv_bfloat16* __restrict__ k_cache,
                                                              const __nv_bfloat16* __restrict__ v_cache,
                                                              const long long* __restrict__ positions, __nv_bfloat16* __restrict__ out,
                                                              int Hq, int Hkv, int max_len, float scale, float* __restrict__ part,
                                                              unsigned int* __restrict__ tickets) {
    constexpr int D = HD / 8;                                 // dims per lane
    __shared__ float sm_m[ATT_SLOTS], sm_l[ATT_SLOTS], sm_acc[ATT_SLOTS][HD];
    __shared__ bool is_last;
    const int bh = blockIdx.x, b = bh / Hq, h = bh - b * Hq, hk = h / (Hq / Hkv);
    const int splits = gridDim.y, split = blockIdx.y;
    const int slot = threadIdx.x >> 3, sub = threadIdx.x & 7;
    pdl_launch_dependents();
    pdl_wait();                                       // q and the newest cache row are the predecessor's output
    long long n_keys = positions[b] + 1;
    if (n_keys > max_len) n_keys = max_len;
    if (n_keys < 0) n_keys = 0;
    const int per = (int)((n_keys + splits - 1) / splits);
    const int j0 = split * per, j1 = (int)min((long long)(j0 + per), n_keys);

    float qf[D];
    {
        const __nv_bfloat16* qp = q + (size_t)b * q_row_stride + (size_t)h * HD + sub * D;
#pragma unroll
        for (int d = 0; d < D; d += 2) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(qp + d);
            qf[d] = bf_lo(w) * scale; qf[d + 1] = bf_hi(w) * scale;
        }
    }
    const __nv_bfloat16* kb = k_cache + ((size_t)b * Hkv + hk) * (size_t)max_len * HD + sub * D;
    const __nv_bfloat16* vb = v_cache + ((size_t)b * Hkv + hk) * (size_t)max_len * HD + sub * D;
    const unsigned int slot_mask = 0xffu << (8 * (slot & 3));
    float mx = -INFINITY, l = 0.0f, acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.0f;
    // KPI keys per slot in flight: the K and V rows of all of them are requested before any arithmetic (the kernel is a
    // chain of memory latencies otherwise; a split covers about 64 keys, i.e. one such round per slot).  A key beyond the
    // range reads key j1-1 again and gets weight zero.
    constexpr int KPI = 4;
    for (int j = j0 + slot; j < j1; j += KPI * ATT_SLOTS) {
        uint4 kq[KPI][D / 8], vq[KPI][D / 8];
        bool on[KPI];
#pragma unroll
        for (int u = 0; u < KPI; ++u) {
            const int ju = j + u * ATT_SLOTS;
            on[u] = ju < j1;
            const size_t row = (size_t)(on[u] ? ju : j1 - 1) * HD;
#pragma unroll
            for (int d = 0; d < D / 8; ++d) {
                kq[u][d] = __ldg(reinterpret_cast<const uint4*>(kb + row) + d);
                vq[u][d] = __ldg(reinterpret_cast<const uint4*>(vb + row) + d);
            }
        }
        float sc[KPI];
#pragma unroll
        for (int u = 0; u < KPI; ++u) {
            float a = 0.0f;
#pragma unroll
            for (int d = 0; d < D / 8; ++d) {
                const uint32_t w[4] = {kq[u][d].x, kq[u][d].y, kq[u][d].z, kq[u][d].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) { a = fmaf(qf[d * 8 + 2 * e], bf_lo(w[e]), a); a = fmaf(qf[d * 8 + 2 * e + 1], bf_hi(w[e]), a); }
            }
            // the four key slots of a warp run different numbers of iterations: only this slot's 8 lanes take part
            a += __shfl_xor_sync(slot_mask, a, 1); a += __shfl_xor_sync(slot_mask, a, 2); a += __shfl_xor_sync(slot_mask, a, 4);
            sc[u] = on[u] ? a : -INFINITY;
        }
        float mn = mx;
#pragma unroll
        for (int u = 0; u < KPI; ++u) mn = fmaxf(mn, sc[u]);
        const float corr = __expf(mx - mn);
        float pw[KPI];
        l *= corr;
#pragma unroll
        for (int u = 0; u < KPI; ++u) { pw[u] = on[u] ? __expf(sc[u] - mn) : 0.0f; l += pw[u]; }
#pragma unroll
        for (int d = 0; d < D; ++d) acc[d] *= corr;
#pragma unroll
        for (int u = 0; u < KPI; ++u) {
#pragma unroll
            for (int d = 0; d < D / 8; ++d) {
                const uint32_t w[4] = {vq[u][d].x, vq[u][d].y, vq[u][d].z, vq[u][d].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[d * 8 + 2 * e] = fmaf(pw[u], bf_lo(w[e]), acc[d * 8 + 2 * e]);
                    acc[d * 8 + 2 * e + 1] = fmaf(pw[u], bf_hi(w[e]), acc[d * 8 + 2 * e + 1]);
                }
            }
        }
        mx = mn;
    }
    // combine the 16 key slots of the CTA
    if (sub == 0) { sm_m[slot] = mx; sm_l[slot] = l; }
#pragma unroll
    for (int d = 0; d < D; ++d) sm_acc[slot][sub * D + d] = acc[d];
    __syncthreads();
    float* my = part + ((size_t)bh * splits + split) * (HD + 2);
    if (threadIdx.x < HD) {
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < ATT_SLOTS; ++s2) M = fmaxf(M, sm_m[s2]);
        float L = 0.0f, a = 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < ATT_SLOTS; ++s2) {
            const float w = (sm_m[s2] == -INFINITY) ? 0.0f : __expf(sm_m[s2] - M);
            L = fmaf(sm_l[s2], w, L); a = fmaf(sm_acc[s2][threadIdx.x], w, a);
        }
        if (splits == 1) {
            out[(size_t)b * Hq * HD + (size_t)h * HD + threadIdx.x] = __float2bfloat16_rn(L > 0.0f ? a / L : 0.0f);
        } else {
            my[threadIdx.x] = a;
            if (threadIdx.x == 0) { my[HD] = M; my[HD + 1] = L; }
        }
    }
    if (splits == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(tickets + bh, 1u);
        is_last = (t == (unsigned int)splits - 1u);
        if (is_last) tickets[bh] = 0u;                          // leave the counter as it was found
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < HD) {
        const float* base = part + (size_t)bh * splits * (HD + 2);
        float M = -INFINITY;
        for (int s2 = 0; s2 < splits; ++s2) M = fmaxf(M, __ldcg(base + (size_t)s2 * (HD + 2) + HD));
        float L = 0.0f, a = 0.0f;
        for (int s2 = 0; s2 < splits; ++s2) {
            const float ms = __ldcg(base + (size_t)s2 * (HD + 2) + HD);
            const float w = (ms == -INFINITY) ? 0.0f : __expf(ms - M);
            L = fmaf(__ldcg(base + (size_t)s2 * (HD + 2) + HD + 1), w, L);
            a = fmaf(__ldcg(base + (size_t)s2 * (HD + 2) + threadIdx.x), w, a);
        }
        out[(size_t)b * Hq * HD + (size_t)h * HD + threadIdx.x] = __float2bfloat16_rn(L > 0.0f ? a / L : 0.0f);
    }
}

// ---------------------------------------------------------------------------------------------
// act[m, i] = silu(gu[m, i]) * gu[m, I + i]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_silu_mul(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                                  int64_t M, int I, int hf_rounding) {
    const int64_t vec_per_row = I / 8, total = M * vec_per_row;
    pdl_launch_dependents();
    pdl_wait();                                       // gate | up is the predecessor's output
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = v / vec_per_row, c = v - m * vec_per_row;
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gu + m * 2 * (int64_t)I) + c);
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(gu + m * 2 * (int64_t)I + I) + c);
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = bf_lo(gw[j]), g1 = bf_hi(gw[j]);
            float s0 = g0 / (1.0f + expf(-g0)), s1 = g1 / (1.0f + expf(-g1));
            if (hf_rounding) { s0 = bf16r(s0); s1 = bf16r(s1); }
            o[j] = pack_bf2(__fmul_rn(s0, bf_lo(uw[j])), __fmul_rn(s1, bf_hi(uw[j])));
        }
        reinterpret_cast<uint4*>(act + m * (int64_t)I)[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---------------------------------------------------------------------------------------------
// End of a greedy decode step in one launch: tok[b] = argmax_v logits[b, v] (the first maximum, NaN counts as the
// largest value, as torch.argmax), positions[b] += 1, h[b, :] = embed[tok[b], :] (the next step's input row).
// One CTA per sequence; a thread walks its vectors in ascending order, so "first" survives the reduction by
// preferring the smaller index among equal values.
// ---------------------------------------------------------------------------------------------
constexpr int AM_THREADS = 1024;
__device__ __forceinline__ bool am_better(float v, int i, float bv, int bi) {
    const bool vn = v != v, bn = bv != bv;
    if (vn != bn) return vn;
    if (!vn && v != bv) return v > bv;
    return i < bi;
}
__global__ void __launch_bounds__(AM_THREADS) k_argmax_embed(const __nv_bfloat16* __restrict__ logits, int64_t logits_stride, int V,
                                                             int vec, const __nv_bfloat16* __restrict__ embed, int D,
                                                             long long* __restrict__ tok, long long* __restrict__ positions,
                                                             __nv_bfloat16* __restrict__ h) {
    __shared__ float sv[AM_THREADS / 32];
    __shared__ int si[AM_THREADS / 32];
    __shared__ int winner;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();                                       // the logits are the predecessor's output
    const __nv_bfloat16* row = logits + (size_t)b * logits_stride;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (vec) {                                        // rows start on 16-byte boundaries and hold whole vectors
        for (int v = tid; v < V / 8; v += AM_THREADS) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + v);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = bf_lo(w[j]), hi = bf_hi(w[j]);
                if (am_better(lo, v * 8 + 2 * j, bv, bi)) { bv = lo; bi = v * 8 + 2 * j; }
                if (am_better(hi, v * 8 + 2 * j + 1, bv, bi)) { bv = hi; bi = v * 8 + 2 * j + 1; }
            }
        }
    } else {
        for (int v = tid; v < V; v += AM_THREADS) {
            const float x = __bfloat162float(row[v]);
            if (am_better(x, v, bv, bi)) { bv = x; bi = v; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (am_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = sv[lane]; bi = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (am_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            winner = bi;
            tok[b] = bi;
            if (positions) positions[b] += 1;
        }
    }
    __syncthreads();
    if (!embed) return;
    const uint4* src = reinterpret_cast<const uint4*>(embed + (size_t)winner * D);
    uint4* dst = reinterpret_cast<uint4*>(h + (size_t)b * D);
    for (int v = tid; v < D / 8; v += AM_THREADS) dst[v] = __ldg(src + v);
}

static inline bool al16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace lq

using namespace lq;

extern "C" {

int lq_add_rmsnorm(void* h, const void* delta, const void* gamma, float eps, void* y, int64_t M, int64_t K, int hf_rounding,
                   lq_stream_t stream) {
    if (!h || !gamma || !y || !al16p(h) || !al16p(gamma) || !al16p(y) || (delta && !al16p(delta))) return LQ_EINVAL;
    if (M < 0 || K <= 0 || (K % 8) != 0 || M >= (1ll << 31) || K >= (1ll << 24)) return LQ_EUNSUPPORTED;
    if (M == 0) return LQ_OK;
    { int rc = ensure_device_for(h); if (rc) return rc; }
    const int vpt = (int)((K / 8 + NORM_THREADS - 1) / NORM_THREADS);
#define LQ_NORM_ARGS dim3((unsigned)M), NORM_THREADS, 0, (cudaStream_t)stream, (__nv_bfloat16*)h, (const __nv_bfloat16*)delta, \
                     (const __nv_bfloat16*)gamma, eps, (__nv_bfloat16*)y, (int)K, hf_rounding
    if (vpt <= 1) launch_pdl(k_add_rmsnorm_r<1>, LQ_NORM_ARGS);
    else if (vpt <= 2) launch_pdl(k_add_rmsnorm_r<2>, LQ_NORM_ARGS);
    else if (vpt <= 4) launch_pdl(k_add_rmsnorm_r<4>, LQ_NORM_ARGS);
    else if (vpt <= 6) launch_pdl(k_add_rmsnorm_r<6>, LQ_NORM_ARGS);
    else launch_pdl(k_add_rmsnorm, LQ_NORM_ARGS);
#undef LQ_NORM_ARGS
    return check_launch("k_add_rmsnorm");
}

int lq_rope_kv_store(void* qkv, const int64_t* positions, const float* inv_freq, void* k_cache, void* v_cache, int64_t M,
                     int tokens_per_seq, int Hq, int Hkv, int hd, int64_t max_len, int hf_rounding, lq_stream_t stream) {
    if (!qkv || !positions || !inv_freq || !k_cache || !v_cache) return LQ_EINVAL;
    if (M < 0 || tokens_per_seq < 1 || Hq < 1 || Hkv < 1 || (Hq % Hkv) != 0 || hd < 8 || hd > 512 || (hd % 4) != 0 || max_len < 1 ||
        max_len >= (1ll << 31) || M >= (1ll << 31) || Hq + 2 * Hkv > 65535)
        return LQ_EUNSUPPORTED;
    if (M == 0) return LQ_OK;
    { int rc = ensure_device_for(qkv); if (rc) return rc; }
    dim3 grid((unsigned)M, (unsigned)(Hq + 2 * Hkv));
    launch_pdl(k_rope_kv_store, grid, (unsigned)(hd / 2), 0, (cudaStream_t)stream, (__nv_bfloat16*)qkv, (const long long*)positions, inv_freq,
               (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tokens_per_seq, Hq, Hkv, hd, (int)max_len, hf_rounding);
    return check_launch("k_rope_kv_store");
}

static int attn_splits(int64_t B, int Hq, int64_t max_len) {
    const int64_t ctas = B * Hq;
    int64_t s = (4 * (int64_t)sm_count() + ctas - 1) / ctas;      // about four CTAs per SM in flight
    const int64_t cap = (max_len + 63) / 64;                        // at least 64 keys (two rounds of the 16 slots x 2) per split
    if (s > cap) s = cap;
    if (s > 32) s = 32;
    if (s < 1) s = 1;
    return (int)s;
}

size_t lq_decode_attention_workspace_bytes(int64_t B, int Hq, int hd, int64_t max_len) {
    if (B <= 0 || Hq <= 0 || hd <= 0 || max_len <= 0) return 0;
    const int s = attn_splits(B, Hq, max_len);
    return (size_t)B * Hq * ((size_t)s * (hd + 2) * sizeof(float) + sizeof(unsigned int));
}

int lq_decode_attention(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache, const int64_t* positions,
                        void* out, int64_t B, int Hq, int Hkv, int hd, int64_t max_len, float scale, void* workspace,
                        size_t workspace_bytes, lq_stream_t stream) {
    if (!q || !k_cache || !v_cache || !positions || !out || !al16p(q) || !al16p(k_cache) || !al16p(v_cache)) return LQ_EINVAL;
    if (B < 0 || Hq < 1 || Hkv < 1 || (Hq % Hkv) != 0 || (hd != 64 && hd != 128) || max_len < 1 || max_len >= (1ll << 31) ||
        B * Hq >= (1ll << 31) || (q_row_stride % 8) != 0)
        return LQ_EUNSUPPORTED;
    if (B == 0) return LQ_OK;
    { int rc = ensure_device_for(q); if (rc) return rc; }
    const int splits = attn_splits(B, Hq, max_len);
    float* part = nullptr; unsigned int* tickets = nullptr;
    if (splits > 1) {
        if (!workspace || workspace_bytes < lq_decode_attention_workspace_bytes(B, Hq, hd, max_len) || !al16p(workspace)) return LQ_EWORKSPACE;
        part = (float*)workspace;
        tickets = (unsigned int*)(part + (size_t)B * Hq * splits * (hd + 2));
    }
    dim3 grid((unsigned)(B * Hq), (unsigned)splits);
    cudaStream_t st = (cudaStream_t)stream;
    if (hd == 128)
        launch_pdl(k_decode_attn<128>, grid, (unsigned)ATT_THREADS, 0, st, (const __nv_bfloat16*)q, (int)q_row_stride, (const __nv_bfloat16*)k_cache,
                   (const __nv_bfloat16*)v_cache, (const long long*)positions, (__nv_bfloat16*)out, Hq, Hkv, (int)max_len, scale, part, tickets);
    else
        launch_pdl(k_decode_attn<64>, grid, (unsigned)ATT_THREADS, 0, st, (const __nv_bfloat16*)q, (int)q_row_stride, (const __nv_bfloat16*)k_cache,
                   (const __nv_bfloat16*)v_cache, (const long long*)positions, (__nv_bfloat16*)out, Hq, Hkv, (int)max_len, scale, part, tickets);
    return check_launch("k_decode_attn");
}

int lq_argmax_embed(const void* logits, int64_t logits_stride, int64_t B, int64_t V, const void* embed, int64_t D, int64_t* tok,
                    int64_t* positions, void* h, lq_stream_t stream) {
    if (!logits || !tok || (embed && (!h || !al16p(embed) || !al16p(h)))) return LQ_EINVAL;
    if (B < 0 || V < 1 || V >= (1ll << 31) - 8 || B >= (1ll << 31) || logits_stride < V || (embed && (D < 8 || (D % 8) != 0 || D >= (1ll << 31))))
        return LQ_EUNSUPPORTED;
    if (B == 0) return LQ_OK;
    { int rc = ensure_device_for(logits); if (rc) return rc; }
    const int vec = al16p(logits) && (logits_stride % 8) == 0 && (V % 8) == 0;
    launch_pdl(k_argmax_embed, dim3((unsigned)B), (unsigned)AM_THREADS, 0, (cudaStream_t)stream, (const __nv_bfloat16*)logits,
               logits_stride, (int)V, vec, (const __nv_bfloat16*)embed, (int)D, (long long*)tok, (long long*)positions,
               (__nv_bfloat16*)h);
    return check_launch("k_argmax_embed");
}

int lq_silu_mul(const void* gate_up, void* act, int64_t M, int64_t I, int hf_rounding, lq_stream_t stream) {
    if (!gate_up || !act || !al16p(gate_up) || !al16p(act)) return LQ_EINVAL;
    if (M < 0 || I <= 0 || (I % 8) != 0 || I >= (1ll << 30)) return LQ_EUNSUPPORTED;
    if (M == 0) return LQ_OK;
    { int rc = ensure_device_for(gate_up); if (rc) return rc; }
    const int64_t total = M * (I / 8);
    int64_t g = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (g > cap) g = cap;
    launch_pdl(k_silu_mul, dim3((unsigned)g), 256u, 0, (cudaStream_t)stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, M, (int)I, hf_rounding);
    return check_launch("k_silu_mul");
}

}  // extern "C"
