// Issue-rate microbenchmark of tcgen05.mma (sm_100a): the measured tensor-core ceilings the GEMM rooflines are
// quoted against.  One CTA per SM issues a long run of 128 x N x (32 bytes of k) MMAs on operands that stay
// resident in shared memory (optionally the A operand in tensor memory), rotating over `n_acc` independent
// accumulators, and reports the cycles the run took.  kind::i8 gives the int8 peak that the A8W8 GEMM is compared
// with; running it with one accumulator against several shows whether an MMA's time depends on the previous MMA
// into the same accumulator.
//
// No counterpart in the reference.  The kernel reads no global memory and writes 8 bytes per CTA.
#include "lq_common.cuh"
#include "lq_tc.cuh"

namespace lq {

constexpr int PROBE_MAX_CTAS = 512;
__device__ unsigned long long g_probe_cycles[PROBE_MAX_CTAS];
__device__ int g_probe_status;

struct ProbeCtl {
    uint64_t done;
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int PROBE_A_BYTES = 128 * 128;      // 128 rows x 128 bytes of k (4 MMAs deep), 128B-swizzled K-major
constexpr int PROBE_B_BYTES = 256 * 128;      // up to 256 rows
constexpr int PROBE_SMEM = PROBE_A_BYTES + PROBE_B_BYTES + 1024 + 64;
constexpr int PROBE_TA_COL0 = 256;            // A operand in tensor memory: 32 columns from here (accumulators use 0..255)

template <bool I8>
__global__ void __launch_bounds__(128, 1) k_mma_probe(int n, int n_acc, int n_mma, int a_in_tmem) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    ProbeCtl* ctl = reinterpret_cast<ProbeCtl*>(smem + PROBE_A_BYTES + PROBE_B_BYTES);
    volatile int* abort_flag = &ctl->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // finite operand values: bf16 in [2^-7, 2^-6) / small int8
    for (int i = threadIdx.x; i < (PROBE_A_BYTES + PROBE_B_BYTES) / 4; i += blockDim.x) {
        const uint32_t h = (uint32_t)i * 2654435761u;
        reinterpret_cast<uint32_t*>(smem)[i] = I8 ? (h & 0x07070707u) : (0x3c003c00u | (h & 0x007f007fu));
    }
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&ctl->done), 1);
        ctl->abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async();
    if (warp == 0) { tmem_alloc(smem_u32(&ctl->tmem_base), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    if (a_in_tmem) {      // every warp fills its lane quarter of the A slot
        const uint32_t a = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)PROBE_TA_COL0;
        const uint32_t v = 0x3c003c00u | (uint32_t)(lane & 0x7f);
        for (int c = 0; c < 32; c += 8) tmem_st8(a + (uint32_t)c, make_uint4(v, v + 1, v + 2, v + 3), make_uint4(v, v + 1, v + 2, v + 3));
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp == 1) {
        // The whole warp runs the loop and one elected lane issues: the operands of tcgen05.mma then stay warp-uniform.
        // (Issued from inside an `if (lane == 0)` the same loop measures the issuing thread, ~115 cycles per MMA, not
        // the tensor pipe.)
        const bool leader = elect_one_sync();
        const uint32_t idesc = make_idesc(I8, false, n);
        const uint64_t a_desc = make_smem_desc(smem_u32(smem), 16, 1024);
        const uint64_t b_desc = make_smem_desc(smem_u32(smem + PROBE_A_BYTES), 16, 1024);
        const long long t0 = clock64();
        int acc = 0;
        for (int i = 0; i < n_mma; i += 4) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t d = tmem_base + (uint32_t)(acc * n);
                const uint32_t accumulate = (i + kk >= n_acc) ? 1u : 0u;
                if (leader) {
                    if (!I8 && a_in_tmem) umma_ta(d, tmem_base + (uint32_t)(PROBE_TA_COL0 + kk * 8), b_desc + (uint64_t)(kk * 2), idesc, accumulate);
                    else umma<I8>(d, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2), idesc, accumulate);
                }
                if (++acc == n_acc) acc = 0;
            }
        }
        if (leader) umma_commit(smem_u32(&ctl->done));
        mbar_wait(smem_u32(&ctl->done), 0, abort_flag);
        const long long t1 = clock64();
        if (leader) {
            if (blockIdx.x < PROBE_MAX_CTAS) g_probe_cycles[blockIdx.x] = (unsigned long long)(t1 - t0);
            if (*abort_flag) atomicExch(&g_probe_status, 1);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace lq

using namespace lq;

extern "C" int lq_mma_issue_rate(int kind, int a_in_tmem, int n, int n_acc, int n_mma, int ctas,
                                 unsigned long long* max_cycles_out, lq_stream_t stream) {
    const bool i8 = kind == LQ_GEMM_A8W8;
    if (n < 16 || n > 256 || (n % 16) != 0 || n_acc < 1 || n_acc * n > 256 || n_mma < 4 || (n_mma % 4) != 0 ||
        n_mma > (1 << 24) || ctas < 1 || ctas > PROBE_MAX_CTAS || (i8 && a_in_tmem))
        return LQ_EINVAL;
    static bool attr_done[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev][i8]) {
        cudaError_t e = i8 ? cudaFuncSetAttribute(k_mma_probe<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM)
                           : cudaFuncSetAttribute(k_mma_probe<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(k_mma_probe)"); return LQ_ECUDA; }
        attr_done[dev][i8] = true;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (i8) k_mma_probe<true><<<ctas, 128, PROBE_SMEM, st>>>(n, n_acc, n_mma, 0);
    else k_mma_probe<false><<<ctas, 128, PROBE_SMEM, st>>>(n, n_acc, n_mma, a_in_tmem);
    int rc = check_launch("k_mma_probe");
    if (rc || !max_cycles_out) return rc;
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { set_cuda_error(e, "cudaStreamSynchronize"); return LQ_ECUDA; }
    static unsigned long long host[PROBE_MAX_CTAS];
    int status = 0;
    e = cudaMemcpyFromSymbol(host, g_probe_cycles, sizeof(unsigned long long) * (size_t)ctas);
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&status, g_probe_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e, "cudaMemcpyFromSymbol(g_probe_cycles)"); return LQ_ECUDA; }
    if (status) { int z = 0; cudaMemcpyToSymbol(g_probe_status, &z, sizeof(int)); return LQ_ETIMEOUT; }
    unsigned long long mx = 0;
    for (int i = 0; i < ctas; ++i) mx = host[i] > mx ? host[i] : mx;
    *max_cycles_out = mx;
    return LQ_OK;
}
