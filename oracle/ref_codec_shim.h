/*
 * Host stand-ins for the CUDA vocabulary used by the kernel bodies of
 * FWkey/latentQ_LLM's utils/cuda_src/multi_random_quant_kernel.cu, so that the
 * reference's own kernel text compiles as plain C++ (g++) and runs one
 * "thread" at a time on the CPU.  No GPU, no launch.
 *
 * TEST INFRASTRUCTURE ONLY (see oracle/build_ref.py).  Nothing of the
 * reference is stored in this file: it only defines what the kernel text
 * needs from the CUDA toolkit.
 *
 *   __global__               -> nothing (the kernels become ordinary functions)
 *   blockIdx/blockDim/threadIdx -> thread-local variables set by the driver;
 *                               the driver runs grids of 1-thread blocks, so the
 *                               `threadIdx.x == 0` staging of the constants into
 *                               shared memory happens for every element
 *   extern __shared__ char shared_mem[40] -> a 40-byte host array (the kernels
 *                               index 40 bytes of it; the reference launcher
 *                               passes 0 dynamic bytes, which is why the kernel
 *                               itself is never launched on a GPU here)
 *   nv_bfloat16              -> 16-bit pattern, conversions round to nearest even
 *                               exactly like __float2bfloat16 / __bfloat162float
 */
#ifndef LQ_REF_CODEC_SHIM_H
#define LQ_REF_CODEC_SHIM_H

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

using std::abs;
using std::round;

#define __global__
#define __shared__
static inline void __syncthreads() {}

struct ref_dim3 { unsigned x, y, z; };
static thread_local ref_dim3 blockIdx = {0, 0, 0}, blockDim = {1, 1, 1}, threadIdx = {0, 0, 0};

alignas(16) char shared_mem[8 * sizeof(float) + 2 * sizeof(int)];

struct nv_bfloat16 { uint16_t bits; };

static inline float __bfloat162float(nv_bfloat16 h) {
    uint32_t u = (uint32_t)h.bits << 16;
    float f; std::memcpy(&f, &u, 4); return f;
}
static inline nv_bfloat16 __float2bfloat16(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    nv_bfloat16 h;
    if ((u & 0x7fffffffu) > 0x7f800000u) { h.bits = (uint16_t)((u >> 16) | 0x0040u); return h; }
    u += 0x7fffu + ((u >> 16) & 1u);
    h.bits = (uint16_t)(u >> 16);
    return h;
}

#endif
