/*
 * Host driver around the reference's own residual-codec kernel text.
 *
 * TEST INFRASTRUCTURE ONLY.  oracle/build_ref.py extracts, at build time, the
 * kernel definitions (utils/cuda_src/multi_random_quant_kernel.cu:9-334) and
 * the constant set-up lines of the three launchers (:346-351, :364, :385-389)
 * from the reference checkout into oracle/_ref/ *.inc (git-ignored); this file
 * includes them and runs every kernel as a grid of one-thread blocks in a host
 * loop.  What comes out is what the reference's kernels compute, up to the
 * compiler's choice of contracting `a*b+c` into a fused multiply-add: the
 * library is built twice (-ffp-contract=off and -ffp-contract=fast -mfma), the
 * tests record which variant the CUDA library and the C restatement match
 * (nvcc's default is to contract).
 *
 * Inputs must lie in the codec's domain |x| <= 0.5 (a rounding residual always
 * does): outside it the kernels convert a negative float to unsigned, which is
 * defined on the GPU (saturates to 0) but not in host C++.
 */
#include "ref_codec_shim.h"

#include "_ref/kernels.inc"

#define REF_API extern "C" __attribute__((visibility("default")))

template <typename F> static void run_grid(int n, F body) {
    blockDim.x = 1; threadIdx.x = 0;
    for (int tid = 0; tid < n; ++tid) { blockIdx.x = (unsigned)tid; body(); }
}

/* launch_quant (.cu:345-361): x holds 8*n values, overwritten by the 0/1 flags; y gets n words.
 * consts10 (may be NULL) receives c1,c2,c3,b1,b2,t1,t2,v0 as the launcher computed them. */
template <typename T, typename K>
static void quant3(T* x, int* y, const int k1, const float b1, const int k2, const float b2, const int k3, int n,
                   float* consts8, K kernel) {
#include "_ref/launch_quant_consts.inc"
    if (consts8) { consts8[0] = c1; consts8[1] = c2; consts8[2] = c3; consts8[3] = b1; consts8[4] = b2;
                   consts8[5] = (float)t1; consts8[6] = (float)t2; consts8[7] = v0; }
    run_grid(n, [&] { kernel(x, y, c1, b1, t1, c2, b2, t2, c3, n, v0); });
}
REF_API void ref_quant_bf16(uint16_t* x, int* y, int k1, float b1, int k2, float b2, int k3, int n, float* consts8) {
    quant3(reinterpret_cast<nv_bfloat16*>(x), y, k1, b1, k2, b2, k3, n, consts8, quant_kernel_bf);
}
REF_API void ref_quant_f32(float* x, int* y, int k1, float b1, int k2, float b2, int k3, int n, float* consts8) {
    quant3(x, y, k1, b1, k2, b2, k3, n, consts8, quant_kernel2<float>);
}

/* launch_dequant (.cu:384-399) */
template <typename T, typename K>
static void dequant3(const int* y, T* x, const int k1, const float b1, const int k2, const float b2, const int k3,
                     int n, float* consts7, K kernel) {
#include "_ref/launch_dequant_consts.inc"
    if (consts7) { consts7[0] = ic1; consts7[1] = ic2; consts7[2] = ic3; consts7[3] = b1; consts7[4] = b2;
                   consts7[5] = (float)t1; consts7[6] = (float)t2; }
    run_grid(n, [&] { kernel(y, x, ic1, b1, t1, ic2, b2, t2, ic3, n); });
}
REF_API void ref_dequant_bf16(const int* y, uint16_t* x, int k1, float b1, int k2, float b2, int k3, int n,
                              float* consts7) {
    dequant3(y, reinterpret_cast<nv_bfloat16*>(x), k1, b1, k2, b2, k3, n, consts7, dequant_kernel_bf);
}
REF_API void ref_dequant_f32(const int* y, float* x, int k1, float b1, int k2, float b2, int k3, int n,
                             float* consts7) {
    dequant3(y, x, k1, b1, k2, b2, k3, n, consts7, dequant_kernel2<float>);
}

/* launch_quant_linear (.cu:363-375) */
REF_API void ref_uniform_quant_bf16(uint16_t* x, int* y, int n) {
#include "_ref/launch_quant_linear_consts.inc"
    run_grid(n, [&] { quant_kernel1_bf(reinterpret_cast<nv_bfloat16*>(x), y, n, v0); });
}
REF_API void ref_uniform_quant_f32(float* x, int* y, int n) {
#include "_ref/launch_quant_linear_consts.inc"
    run_grid(n, [&] { quant_kernel1<float>(x, y, n, v0); });
}
/* launch_quant_linear_s (.cu:377-382) */
REF_API void ref_uniform_quant_s_f32(float* x, int* y, int n) {
    run_grid(n, [&] { quant_kernel0<float>(x, y, n); });
}
/* launch_dequant_linear (.cu:401-412) */
REF_API void ref_uniform_dequant_bf16(int* y, uint16_t* x, int n) {
    run_grid(n, [&] { dequant_kernel1_bf(y, reinterpret_cast<nv_bfloat16*>(x), n); });
}
REF_API void ref_uniform_dequant_f32(int* y, float* x, int n) {
    run_grid(n, [&] { dequant_kernel1<float>(y, x, n); });
}
