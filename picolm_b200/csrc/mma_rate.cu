// A measuring kernel, not part of any model step: how many cycles one tcgen05.mma (bf16, K = 16,
// cta_group::1) takes, by tile shape, by where the A operand lives (shared or tensor memory), by the
// layout of B (K-major or MN-major) and by how many CTAs of an SM issue at the same time.  One thread
// of each CTA issues a long run of MMAs into one accumulator and waits (bounded) for a single commit;
// nothing is loaded: the operands are whatever shared and tensor memory hold.  The tile shapes of the
// tcgen05 kernels in this folder were chosen against these figures.
#include "tc_common.cuh"

using namespace plm_tc;

namespace {

constexpr int A_BYTES = 128 * 128;            // 128 rows of 64 bf16
constexpr int B_BYTES = 256 * 128;            // up to 256 rows (K-major) or 4 blocks of 64 columns (MN-major)
constexpr int TMEM_COLS = 256;                // accumulator at column 0, the A operand (N <= 128 then) at column 192
constexpr size_t SMEM = A_BYTES + B_BYTES + 1024;

__device__ __forceinline__ void mma_a_tmem(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// B with its N dimension contiguous, 128-byte swizzle: 8-row groups 1024 bytes apart, 64-column blocks 8192
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__host__ __device__ constexpr uint32_t idesc_of(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(128, 2)
mma_rate_kernel(int a_tmem, int b_mn, int m, int n, int reps, long long* __restrict__ cycles, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bar;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint32_t* words = reinterpret_cast<uint32_t*>(smem_raw + (base - smem_u32(smem_raw)));
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x) words[i] = 0x3c003c00u;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t a_smem = base, b_smem = base + A_BYTES;
        const uint32_t idesc = idesc_of(m, n, b_mn != 0);
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {                        // the four K = 16 steps of a 64-element block
                const uint64_t bd = b_mn ? desc_mn(b_smem + k * 2048) : smem_desc_sw128(b_smem) + (uint64_t)(k * 2);
                if (a_tmem) mma_a_tmem(tmem, tmem + 192 + k * 8, bd, idesc, 1u);
                else tc_mma_bf16(tmem, smem_desc_sw128(a_smem) + (uint64_t)(k * 2), bd, idesc, 1u);
            }
        }
        tc_commit(smem_u32(&bar));
        const bool ok = mbar_wait(smem_u32(&bar), 0, status, 1);
        const long long t1 = clock64();
        if (blockIdx.x == 0) cycles[0] = ok ? t1 - t0 : -1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

// Launches `ctas` CTAs (148 is one an SM, 296 two) that each issue 4 * reps MMAs of m x n x 16;
// cycles[0] (device, int64) gets the cycles CTA 0 took from its first issue to the commit's arrival,
// -1 if the wait ran out.  m in {64, 128}, n a multiple of 16 up to 256 (128 with A in tensor memory).
extern "C" int plm_mma_rate(int a_tmem, int b_mn, int m, int n, int reps, int ctas, long long* cycles, int* status,
                            cudaStream_t stream) {
    if ((m != 64 && m != 128) || n < 16 || n > (a_tmem ? 128 : 256) || n % 16 || reps <= 0 || ctas <= 0) return PLM_ERR_SHAPE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    mma_rate_kernel<<<ctas, 128, SMEM, stream>>>(a_tmem, b_mn, m, n, reps, cycles, status);
    return plm_status_of(cudaGetLastError());
}
