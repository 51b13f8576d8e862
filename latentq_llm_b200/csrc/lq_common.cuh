// Shared device/host helpers for liblatentq (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "latentq.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "liblatentq targets sm_100a only"
#endif

namespace lq {

// ---- host-side error plumbing ------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);
int check_launch(const char* where);  // cudaGetLastError -> LQ_OK / LQ_ECUDA
int sm_count();                       // cached per current device
// Makes the device that owns `device_ptr` current on the calling thread if the thread has no CUDA context yet
// (worker threads such as an autograd engine thread start without one; launching from them would otherwise
// target device 0, and tensor-map encoding fails outright).  No-op when a context is already current.
int ensure_device_for(const void* device_ptr);

// ---- programmatic dependent launch (decode chain) -------------------------------------------------
// A decode step is a chain of short launches in which every kernel consumes its predecessor's output.  Inside such a
// chain (lq_decode_chain(1)) kernels are launched with programmatic stream serialization: a kernel signals
// launch_dependents early, so that its successor's launch latency (and, for the GEMMs, the first round of weight loads)
// overlaps its own run, and every kernel reads what a predecessor may have written only after pdl_wait(), which returns
// once the predecessor grid has completed and its writes are visible.  Outside a chain the attribute is off and both
// instructions are no-ops: a caller whose previous kernel wrote the WEIGHTS (an optimizer step followed by a forward)
// must not have those read early.
bool decode_chain_enabled();
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
template <typename... KArgs, typename... Args>
static inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(block); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = decode_chain_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- numeric helpers ------------------------------------------------------------
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <bool BF> __device__ __forceinline__ float rnd(float x) { return BF ? bf16r(x) : x; }
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// three_fold_curve_4bit (utils/quant.py:708-716) as the constants the reference launchers derive
// (utils/cuda_src/multi_random_quant_kernel.cu:345-351, 384-389).
struct Curve {
    float c1, c2, c3, ic1, ic2, ic3, b1, b2, t1, t2;
};
inline Curve make_curve(int k1, float b1, int k2, float b2, int k3) {
    Curve c;
    c.c1 = (float)k1 / b1;
    c.c2 = (float)k2 / (b2 - b1);
    c.c3 = (float)((double)k3 / (0.5 - (double)b2));
    c.ic1 = b1 / (float)k1;
    c.ic2 = (b2 - b1) / (float)k2;
    c.ic3 = (float)((0.5 - (double)b2) / (double)k3);
    c.b1 = b1; c.b2 = b2; c.t1 = (float)k1; c.t2 = (float)(k1 + k2);
    return c;
}
inline Curve curve_for_level(int mu) {
    switch (mu) {
        case 3: return make_curve(2, 0.4330623539159437f, 2, 0.46875f, 4);
        case 2: return make_curve(2, 0.37272211741724515f, 2, 0.4375f, 4);
        case 1: return make_curve(2, 0.2666300266320331f, 2, 0.375f, 4);
        default: return make_curve(2, 0.125f, 2, 0.25f, 4);
    }
}

// |x|*499 + v0, minus its round-half-away integer part (.cu:49-51); `a*b+c` is an FMA under nvcc defaults.
__device__ __forceinline__ float hash_dither(float x, float v0) {
    float v = __fmaf_rn(fabsf(x), 499.0f, v0);
    return __fsub_rn(v, roundf(v));
}
// 3-fold encode of one residual (.cu:52-63). Returns the nibble, sets carry.
__device__ __forceinline__ uint32_t res3_encode(float x, float v, const Curve& c, float& carry) {
    float S = fabsf(x), q;
    if (S < c.b1) {
        q = roundf(__fmaf_rn(x, c.c1, v));
    } else if (S < c.b2) {
        float r = __fadd_rn(roundf(__fmaf_rn(__fsub_rn(S, c.b1), c.c2, v)), c.t1);
        q = (x < 0.0f) ? -r : r;
    } else {
        float r = __fadd_rn(roundf(__fmaf_rn(__fsub_rn(S, c.b2), c.c3, v)), c.t2);
        q = (x < 0.0f) ? -r : r;
    }
    if (q > 7.5f) { carry = 1.0f; return 1u; }
    carry = 0.0f;
    float t = q + 8.0f;
    return (t <= 0.0f) ? 0u : (uint32_t)t;
}
// 3-fold decode of one nibble (.cu:160-169).
__device__ __forceinline__ float res3_decode(uint32_t nib, const Curve& c) {
    float s = (float)((int)nib - 8);
    if (s < -c.t2) return __fmaf_rn(s + c.t2, c.ic3, -c.b2);
    if (s < -c.t1) return __fmaf_rn(s + c.t1, c.ic2, -c.b1);
    if (s <= c.t1) return __fmul_rn(s, c.ic1);
    if (s <= c.t2) return __fmaf_rn(s - c.t1, c.ic2, c.b1);
    return __fmaf_rn(s - c.t2, c.ic3, c.b2);
}

// Philox4x32-10 (Salmon et al., SC'11), same constants as cuRAND.
__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];   // one wide multiply each
        const uint32_t h0 = (uint32_t)(p0 >> 32), l0 = (uint32_t)p0, h1 = (uint32_t)(p1 >> 32), l1 = (uint32_t)p1;
        uint32_t n0 = h1 ^ c[1] ^ k0, n2 = h0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = l1; c[2] = n2; c[3] = l0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}
// Dither of the 8 elements of residual word `word`: 16 random bits each, u = h/65536 - 0.5 (exact).
__device__ __forceinline__ void philox_dither8(uint64_t seed, uint64_t stream_id, uint64_t word, float (&u)[8]) {
    uint32_t c[4] = {(uint32_t)word, (uint32_t)(word >> 32), (uint32_t)stream_id, (uint32_t)(stream_id >> 32)};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        uint32_t h = (k & 1) ? (c[k >> 1] >> 16) : (c[k >> 1] & 0xffffu);
        // (2^23 + h) * 2^-16 - 128.5 == h/65536 - 0.5 with no rounding
        u[k] = __fmaf_rn(__uint_as_float(0x4B000000u | h), 1.0f / 65536.0f, -128.5f);
    }
}

// Correctly rounded a/s from r = RN(1/s): q0 = a*r followed by two FMA residual corrections (the
// refinement CUDA's own division uses).  Valid for normal, mid-range operands; callers fall back to
// __fdiv_rn otherwise.
__device__ __forceinline__ bool fastdiv_ok_scale(float s) {
    float a = fabsf(s);
    return a >= 9.094947e-13f && a <= 1.0995116e12f;  // 2^-40 .. 2^40
}
__device__ __forceinline__ float div_rn(float a, float s, float r, bool scale_ok) {
    float m = fabsf(a);
    if (scale_ok && (m == 0.0f || (m >= 8.6736174e-19f && m <= 1.1529215e18f))) {  // 2^-60 .. 2^60
        float q = __fmul_rn(a, r);
        float e = __fmaf_rn(-q, s, a);
        q = __fmaf_rn(e, r, q);
        e = __fmaf_rn(-q, s, a);
        return __fmaf_rn(e, r, q);
    }
    return __fdiv_rn(a, s);
}

}  // namespace lq
