// out[T, F] = X[T, K] * W[F, K]^T for many tokens (T > 64), the shape of a prompt
// step: a persistent tcgen05 kernel.  One CTA per SM walks over 128 x BN output tiles
// (BN = 256, or 128 for narrow problems); the tokens sit on the 128 TMEM lanes, the
// features on the accumulator columns.  The accumulator has two buffers in tensor
// memory, so the MMA warp runs the next tile's main loop while the epilogue warps read
// the last tile out (tcgen05.ld), convert and store it; the TMA ring keeps running across
// tile boundaries, so there is no pipeline ramp per tile.
//
// This is the reference's matmul_batch, out[b*d + i] = W[i, :] . x[b, :]
// (picolm/tensor.c:2174), and for the SwiGLU epilogue its silu(W_g x) * (W_u x)
// (picolm/model_core.c:3183-3192), for 16-bit weights.
//   EPI_STORE   out = product (fp32 or bf16)
//   EPI_SWIGLU  W's rows come in tiles of 64 gate rows followed by their 64 up rows;
//               out[t, f] = silu(gate) * up, [T, F/2] in bf16
// Warp 0 loads (TMA), warp 1 issues the MMAs and owns the tensor memory, warps 2..5 are the
// epilogue.  Waits on mbarriers are bounded; a wait that runs out records where in `status`
// and the CTA drains and leaves.
#include "tc_common.cuh"

using namespace plm_tc;

namespace {

constexpr int EPI_STORE = 0, EPI_SWIGLU = 1;

__host__ __device__ constexpr int stages_of(int bn) { return bn >= 256 ? 4 : 6; }
__host__ __device__ constexpr size_t wide_smem(int bn) {
    return (size_t)stages_of(bn) * (BM * BK * 2 + bn * BK * 2) + 1024 + 256;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int BN, int EPI, typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    OutT* __restrict__ out, int T, int F, int K, long ldo, int m_tiles, int n_tiles,
                    int* __restrict__ status) {
    constexpr int STAGES = stages_of(BN);
    constexpr uint32_t X_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;                               // two accumulators
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t x_smem = base, w_smem = base + STAGES * X_BYTES;
    const uint32_t bars = w_smem + STAGES * W_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, acc_full0 = bars + 16 * STAGES,
                   acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (acc_empty0 + 16 - raw));
    __shared__ int s_abort;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + BK - 1) / BK;
    const int n_tiles_total = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool waited = false;
            int it = 0;                                                  // K blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, f0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, status, 1)) { s_abort = 1; ok = false; break; }
                    mbar_expect_tx(full0 + 8 * s, X_BYTES + W_BYTES);
                    // weights are written by no kernel of the step: they may be requested at once
                    tma_load_2d(w_smem + s * W_BYTES, &map_w, full0 + 8 * s, kb * BK, f0);
                    if (!waited) { pdl_wait(); waited = true; }         // activations come from the kernel before
                    tma_load_2d(x_smem + s * X_BYTES, &map_x, full0 + 8 * s, kb * BK, m0);
                }
            }
            if (*(volatile int*)&s_abort)
                for (int i = max(0, it - STAGES); i < it; ++i)
                    mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr, 0);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            int it = 0, j = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x, ++j) {
                const int acc = j & 1;
                // the epilogue must have read this accumulator's previous tile out
                if (!mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, status, 2)) { s_abort = 1; ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, status, 2)) { s_abort = 1; ok = false; break; }
                    tc_fence_after();
                    const uint64_t xd = smem_desc_sw128(x_smem + s * X_BYTES);
                    const uint64_t wd = smem_desc_sw128(w_smem + s * W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_bf16(tmem_base + acc * BN, xd + (uint64_t)(k * UMMA_K * 2 / 16),
                                    wd + (uint64_t)(k * UMMA_K * 2 / 16), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);
                }
                tc_commit(acc_full0 + 8 * acc);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        pdl_wait();                                                      // the output may still be in use by an earlier kernel
        int j = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x, ++j) {
            const int acc = j & 1;
            const int m0 = (tile % m_tiles) * BM, f0 = (tile / m_tiles) * BN;
            if (!mbar_wait(acc_full0 + 8 * acc, (j >> 1) & 1, status, 3)) { s_abort = 1; ok = false; break; }
            tc_fence_after();
            const int t = m0 + quarter * 32 + lane;                      // the token row held by this thread
            const uint32_t tacc = tmem_base + lane_bits + acc * BN;
            if (EPI == EPI_SWIGLU) {
#pragma unroll 1
                for (int gq = 0; gq < BN; gq += 128) {
                    if (f0 + gq >= F) break;
#pragma unroll 1
                    for (int cc = 0; cc < 64; cc += 32) {
                        uint32_t gt[32], up[32];
                        tc_ld32(tacc + gq + cc, gt);
                        tc_ld32(tacc + gq + 64 + cc, up);
                        tc_wait_ld();
                        if (t < T) {
                            const int fo = (f0 + gq) / 2 + cc;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                gt[i] = __float_as_uint(swiglu_bf16(__uint_as_float(gt[i]), __uint_as_float(up[i])));
                            OutT* rowp = out + (size_t)t * ldo + fo;
                            if ((((size_t)t * ldo + fo) * sizeof(OutT)) % 16 == 0) {
#pragma unroll
                                for (int i = 0; i < 32; i += 8) store_vec8<OutT>(rowp + i, gt + i);
                            } else {
                                for (int i = 0; i < 32; ++i) rowp[i] = from_f32<OutT>(__uint_as_float(gt[i]));
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (f0 + c >= F) break;
                    uint32_t r[32];
                    tc_ld32(tacc + c, r);
                    tc_wait_ld();
                    if (t < T) {
                        OutT* rowp = out + (size_t)t * ldo + f0 + c;
                        const bool vec = (f0 + c + 32 <= F) && ((((size_t)t * ldo + f0 + c) * sizeof(OutT)) % 16 == 0);
                        if (vec) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) store_vec8<OutT>(rowp + i, r + i);
                        } else {
                            for (int i = 0; i < 32; ++i)
                                if (f0 + c + i < F) rowp[i] = from_f32<OutT>(__uint_as_float(r[i]));
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty0 + 8 * acc);                           // this accumulator may be overwritten
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

template <int BN, int EPI, typename OutT>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, OutT* out, int T, int F, int K, long ldo, int* status,
           cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = wide_smem(BN);
    auto kern = gemm_tc_wide_kernel<BN, EPI, OutT>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = (T + BM - 1) / BM, n_tiles = (F + BN - 1) / BN;
    const int ctas = m_tiles * n_tiles < sm_count() ? m_tiles * n_tiles : sm_count();
    return plm_status_of(launch_pdl(kern, dim3(ctas), dim3(NUM_THREADS), smem, stream, mx, mw, out, T, F, K, ldo, m_tiles,
                                    n_tiles, status));
}

}  // namespace

// out[T, F'] = epilogue(x[T, K] * w[F, K]^T), T > 64, bf16 operands that TMA can address (K and the
// leading dimensions multiples of 8, pointers 16-byte aligned).  epilogue 0: F' = F, out float32
// (out_dtype 0) or bfloat16 (1).  epilogue 1 (SwiGLU): w holds tiles of 64 gate rows followed by their
// 64 up rows (F a multiple of 128), F' = F / 2, out bfloat16.
extern "C" int plm_gemm_tc_wide(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                int K, long ldx, long ldw, long ldo, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && (F % 128 || out_dtype != PLM_BF16)) return PLM_ERR_SHAPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) return PLM_ERR_UNSUPPORTED;
    const int bn = (F >= 2048 && T >= 256) ? 256 : 128;
    CUtensorMap mx, mw;
    int rc;
    if ((rc = make_map(&mx, x, T, K, ldx, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mw, w, F, K, ldw, bn)) != PLM_OK) return rc;
    if (epilogue == EPI_SWIGLU) {
        if (bn == 256) return launch<256, EPI_SWIGLU, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
        return launch<128, EPI_SWIGLU, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
    }
    if (out_dtype == PLM_F32) {
        if (bn == 256) return launch<256, EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
        return launch<128, EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
    }
    if (out_dtype == PLM_BF16) {
        if (bn == 256) return launch<256, EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
        return launch<128, EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
    }
    return PLM_ERR_DTYPE;
}
