// out[T, F] = X[T, K] * W[F, K]^T in bfloat16 with fp32 accumulation on the
// fifth-generation tensor cores: operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), tcgen05.mma issued by one thread,
// the accumulator in tensor memory, read back with tcgen05.ld for the epilogue.
//
// This is the reference's matmul / matmul_batch, out[b*d + i] = W[i, :] . x[b, :]
// with W row-major [out_features, in_features] (picolm/tensor.c:1394-1418,
// picolm/tensor.c:2174), for 16-bit weights (picolm/quant.c:133-153), as one
// tensor-core kernel.
//
// For outside callers with a plain C ABI and at most 64 rows of X (a decode step's
// shapes): plm_gemm_tc takes a caller-provided fp32 workspace, plm_gemm_tc_static
// (gemm_tc_static.h) keeps the workspace inside the library.  The engine itself
// uses gemm_tc_skinny.cu (no workspace at all) and gemm_tc_wide.cu (more rows).
//
// One CTA computes one 128 x BN tile of D = W * X^T: the weights W on the 128 TMEM
// lanes, the tokens X on the BN = 16..64 accumulator columns, so that the step
// streams each weight once with full tiles.  K is split over gridDim.z CTAs so
// that all SMs pull from HBM; the fp32 partials go to the workspace and are
// summed in a fixed order by a second kernel.
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (each reads the TMEM lane quarter warp_id % 4).
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA records
// where in `status`, stops issuing, drains what it has in flight, frees its
// tensor memory and returns.
#include "tc_common.cuh"

using namespace plm_tc;

namespace {

// skinny tiles (bn < 128) keep their ring small enough for two CTAs per SM
__host__ __device__ constexpr int stages_for(int bn) { return 5; }
__host__ __device__ constexpr size_t smem_bytes_for(int bn) {
    return (size_t)stages_for(bn) * (BM * BK * 2 + bn * BK * 2) + 1024 /*alignment slack*/ + 256 /*barriers*/;
}

// P: the weights [p_rows, K], Q: the tokens [q_rows, K], both bf16 K-major, described by
// the tensor maps; out[q, p].
// gridDim = (P tiles, Q tiles, K splits).  With more than one split, OutT is
// float and the CTA writes its partial sum to out + blockIdx.z * split_stride.
template <int BN, typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               OutT* __restrict__ out, int p_rows, int q_rows, int K, long ldo, int kb_per_split, long split_stride,
               int* __restrict__ status) {
    constexpr int STAGES = stages_for(BN);
    constexpr uint32_t P_BYTES = BM * BK * 2, Q_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                       // tiles need 1024-byte alignment
    const uint32_t p_smem = base, q_smem = base + STAGES * P_BYTES;
    const uint32_t bars = q_smem + STAGES * Q_BYTES;                     // full[STAGES], empty[STAGES], tmem_full
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tmem_full = bars + 16 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars + 16 * STAGES + 8 - raw));
    __shared__ int s_abort;

    pdl_launch_dependents();                   // the next kernel may set itself up while this one runs
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * BM, q0 = blockIdx.y * BN;
    const int n_kb_total = (K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(n_kb_total, kb_begin + kb_per_split);
    const int n_kb = kb_end - kb_begin;                                  // >= 1 by construction of the grid

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tmem_full, 1);
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
        // ------------------------------------------------------ TMA producer
        // The weight operand is assumed to be written by no kernel that runs just before this one,
        // so its first ring of loads is issued before pdl_wait(); the activation operand only after it.
        if (lane == 0) {
            const CUtensorMap* w_map = &map_p;
            const CUtensorMap* x_map = &map_q;
            const uint32_t w_smem = p_smem, x_smem = q_smem;
            const uint32_t W_BYTES = P_BYTES, X_BYTES = Q_BYTES;
            const int w_row = p0, x_row = q0;
            const int early = n_kb < STAGES ? n_kb : STAGES;
            for (int i = 0; i < early; ++i) {              // the ring is empty: no wait needed
                mbar_expect_tx(full0 + 8 * i, P_BYTES + Q_BYTES);
                tma_load_2d(w_smem + i * W_BYTES, w_map, full0 + 8 * i, (kb_begin + i) * BK, w_row);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(x_smem + i * X_BYTES, x_map, full0 + 8 * i, (kb_begin + i) * BK, x_row);
            int issued = early;
            for (int i = early; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (*(volatile int*)&s_abort) break;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1, status, 1)) { s_abort = 1; break; }
                mbar_expect_tx(full0 + 8 * s, P_BYTES + Q_BYTES);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(w_smem + s * W_BYTES, w_map, full0 + 8 * s, k, w_row);
                tma_load_2d(x_smem + s * X_BYTES, x_map, full0 + 8 * s, k, x_row);
                issued = i + 1;
            }
            if (*(volatile int*)&s_abort) {
                // drain: every load this thread issued must land before the CTA's shared memory goes away
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr, 0);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (*(volatile int*)&s_abort) { ok = false; break; }
                if (!mbar_wait(full0 + 8 * s, phase, status, 2)) { s_abort = 1; ok = false; break; }
                tc_fence_after();
                const uint64_t pd = smem_desc_sw128(p_smem + s * P_BYTES);
                const uint64_t qd = smem_desc_sw128(q_smem + s * Q_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_bf16(tmem_base, pd + (uint64_t)(k * UMMA_K * 2 / 16), qd + (uint64_t)(k * UMMA_K * 2 / 16),
                                idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty0 + 8 * s);              // the stage is free once these MMAs have read it
            }
            tc_commit(tmem_full);                       // arrives when every MMA issued so far is done
        }
    } else {
        // ----------------------------------------------------------- epilogue
        const int quarter = warp & 3;                   // the TMEM lanes this warp may read
        pdl_wait();                                     // the output may still be in use by an earlier kernel
        const bool ready = mbar_wait(tmem_full, 0, status, 3);
        if (!ready) s_abort = 1;
        tc_fence_after();
        if (ready && !*(volatile int*)&s_abort) {
            const int p = p0 + quarter * 32 + lane;     // row of P held by this thread
            OutT* dst = out + (size_t)blockIdx.z * split_stride;
            constexpr int CHUNK = BN >= 32 ? 32 : 16;
#pragma unroll 1
            for (int c = 0; c < BN; c += CHUNK) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c;
                if (CHUNK == 32) tc_ld32(taddr, r); else tc_ld16(taddr, r);
                tc_wait_ld();
                if (p < p_rows) {
#pragma unroll
                    for (int j = 0; j < CHUNK; ++j) {
                        const int q = q0 + c + j;       // a token; lanes write consecutive features: coalesced
                        if (q < q_rows) dst[(size_t)q * ldo + p] = from_f32<OutT>(__uint_as_float(r[j]));
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (*(volatile int*)&s_abort && lane == 0) {
            // MMAs that were issued still read shared memory and write TMEM: let them finish (bounded)
            mbar_wait(tmem_full, 0, nullptr, 0);
        }
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// out[i] = sum over splits of partial[s][i], in ascending s.  VEC: total is a
// multiple of 4, so every split's slice starts on a 16-byte boundary.
template <typename OutT, bool VEC>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ out, int splits, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    if (VEC) {
        const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
        if (i >= total) return;
        float4 acc = *reinterpret_cast<const float4*>(partial + i);
        for (int s = 1; s < splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)s * total + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        out[i] = from_f32<OutT>(acc.x); out[i + 1] = from_f32<OutT>(acc.y);
        out[i + 2] = from_f32<OutT>(acc.z); out[i + 3] = from_f32<OutT>(acc.w);
    } else {
        const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= total) return;
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) acc += partial[(size_t)s * total + i];
        out[i] = from_f32<OutT>(acc);
    }
}

template <int BN, typename OutT>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, OutT* out, int p_rows, int q_rows, int K, long ldo,
           int splits, int kb_per_split, long split_stride, int* status, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = smem_bytes_for(BN);
    auto kern = gemm_tc_kernel<BN, OutT>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((p_rows + BM - 1) / BM, (q_rows + BN - 1) / BN, splits);
    return plm_status_of(launch_pdl(kern, grid, dim3(NUM_THREADS), smem, stream, mp, mq, out, p_rows, q_rows, K, ldo,
                                    kb_per_split, split_stride, status));
}

template <typename OutT>
int launch_reduce(const float* partial, OutT* out, int splits, size_t total, cudaStream_t stream) {
    if (total % 4 == 0) {
        const size_t threads = total / 4;
        return plm_status_of(launch_pdl(splitk_reduce_kernel<OutT, true>, dim3((unsigned)((threads + 255) / 256)),
                                        dim3(256), 0, stream, partial, out, splits, total));
    }
    return plm_status_of(launch_pdl(splitk_reduce_kernel<OutT, false>, dim3((unsigned)((total + 255) / 256)), dim3(256),
                                    0, stream, partial, out, splits, total));
}

}  // namespace

// Whether plm_gemm_tc takes this problem: bf16 operands whose rows start on
// 16-byte boundaries (TMA's rule: K and the leading dimensions are multiples of 8
// elements, the base pointers 16-byte aligned).
extern "C" int plm_gemm_tc_supported(const void* x, const void* w, int T, int F, int K, long ldx, long ldw) {
    if (T <= 0 || F <= 0 || K <= 0) return 0;
    if (K % 8 || ldx % 8 || ldw % 8) return 0;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return 0;
    return 1;
}

// Number of K splits and fp32 workspace elements that plm_gemm_tc will use for a
// problem.  Fixed by (T, F, K) alone.
extern "C" int plm_gemm_tc_plan(int T, int F, int K, int* splits_out, long* workspace_elems) {
    int splits = 1;
    if (T <= 64) {
        const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
        const int tiles = ((F + BM - 1) / BM) * ((T + bn - 1) / bn);
        const int n_kb = (K + BK - 1) / BK;
        int want = (2 * PLM_SM_COUNT + tiles - 1) / tiles;              // about two CTAs per SM
        if (want > n_kb / 2) want = n_kb / 2;                  // at least two K blocks per split
        if (want < 1) want = 1;
        const int per = (n_kb + want - 1) / want;
        splits = (n_kb + per - 1) / per;
    }
    *splits_out = splits;
    *workspace_elems = splits > 1 ? (long)splits * T * F : 0;
    return PLM_OK;
}

// out[T, F] (out_dtype, leading dimension ldo) = x[T, K] * w[F, K]^T for T <= 64.
// `w` must not be written by the kernel that runs just before this one on the stream
// (its first tiles are requested before that kernel has finished).
// `workspace` must hold the elements that plm_gemm_tc_plan reports; `status` is
// a device int that is 0 unless a bounded wait ran out (then 1, 2 or 3: producer,
// MMA issuer, epilogue).
extern "C" int plm_gemm_tc(const void* x, const void* w, void* out, int out_dtype, int T, int F, int K, long ldx,
                           long ldw, long ldo, float* workspace, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (!plm_gemm_tc_supported(x, w, T, F, K, ldx, ldw)) return PLM_ERR_ALIGN;
    if (out_dtype != PLM_F32 && out_dtype != PLM_BF16) return PLM_ERR_DTYPE;
    if (T > 64) return PLM_ERR_SHAPE;                      // more rows belong to plm_gemm_tc_wide
    CUtensorMap mp, mq;
    int rc;
    // skinny: weights on the TMEM lanes, tokens on the accumulator columns
    int splits;
    long ws_elems;
    plm_gemm_tc_plan(T, F, K, &splits, &ws_elems);
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    const int n_kb = (K + BK - 1) / BK;
    const int per = (n_kb + splits - 1) / splits;
    if ((rc = make_map(&mp, w, F, K, ldw, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mq, x, T, K, ldx, bn)) != PLM_OK) return rc;
    if (splits > 1) {
        if (!workspace) return PLM_ERR_SHAPE;
        const long stride = (long)T * F;
        if (ldo != F) return PLM_ERR_SHAPE;
        if (bn == 16) rc = launch<16, float>(mp, mq, workspace, F, T, K, F, splits, per, stride, status, stream);
        else if (bn == 32) rc = launch<32, float>(mp, mq, workspace, F, T, K, F, splits, per, stride, status, stream);
        else rc = launch<64, float>(mp, mq, workspace, F, T, K, F, splits, per, stride, status, stream);
        if (rc != PLM_OK) return rc;
        return out_dtype == PLM_F32 ? launch_reduce<float>(workspace, (float*)out, splits, (size_t)stride, stream)
                                    : launch_reduce<bf16>(workspace, (bf16*)out, splits, (size_t)stride, stream);
    }
    if (out_dtype == PLM_F32) {
        if (bn == 16) return launch<16, float>(mp, mq, (float*)out, F, T, K, ldo, 1, n_kb, 0, status, stream);
        if (bn == 32) return launch<32, float>(mp, mq, (float*)out, F, T, K, ldo, 1, n_kb, 0, status, stream);
        return launch<64, float>(mp, mq, (float*)out, F, T, K, ldo, 1, n_kb, 0, status, stream);
    }
    if (bn == 16) return launch<16, bf16>(mp, mq, (bf16*)out, F, T, K, ldo, 1, n_kb, 0, status, stream);
    if (bn == 32) return launch<32, bf16>(mp, mq, (bf16*)out, F, T, K, ldo, 1, n_kb, 0, status, stream);
    return launch<64, bf16>(mp, mq, (bf16*)out, F, T, K, ldo, 1, n_kb, 0, status, stream);
}

// ------------------------------------------------- the entry point that allocates nothing
// See gemm_tc_static.h for whom this is and what it costs.  The partial sums of the split-K
// product go to this file-scope array instead of a caller-provided workspace.
#include "gemm_tc_static.h"

static __device__ __align__(256) float plm_static_scratch[PLM_GEMM_TC_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
// Device address of plm_static_scratch on each device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use: the address comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
float* g_scratch_ptr[MAX_DEVICES];
}  // namespace

extern "C" const char* plm_gemm_tc_static_strerror(int code) {
    switch (code) {
        case PLM_OK: return "ok";
        case PLM_ERR_DTYPE: return "unsupported element type (out_dtype must be 0 = float32 or 1 = bfloat16)";
        case PLM_ERR_SHAPE: return "bad shape or leading dimension (ldo must equal F when K is split)";
        case PLM_ERR_ALIGN: return "operands are not addressable by TMA (K and the leading dimensions must be "
                                   "multiples of 8, the pointers 16-byte aligned)";
        case PLM_ERR_UNSUPPORTED: return "the driver does not offer cuTensorMapEncodeTiled";
        case PLM_ERR_SCRATCH_TOO_SMALL: return "the partial sums of this problem (splits * T * F floats) exceed the "
                                               "library's fixed scratch array (PLM_GEMM_TC_STATIC_SCRATCH_FLOATS)";
        case PLM_ERR_SCRATCH_SETUP: return "the device address of the library's scratch array could not be obtained";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown refusal";
    }
}

extern "C" int plm_gemm_tc_static(const void* x, const void* w, void* out, int out_dtype, int T, int F, int K, long ldx,
                                  long ldw, long ldo, int* status, cudaStream_t stream) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return PLM_ERR_SCRATCH_SETUP;
    if (g_scratch_ptr[dev] == nullptr) {                 // set-up, once per device, that device being current
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, plm_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return PLM_ERR_SCRATCH_SETUP;
        g_scratch_ptr[dev] = p;
    }
    if (T <= 0 || F <= 0) return PLM_OK;
    int splits = 1;
    long need = 0;
    plm_gemm_tc_plan(T, F, K, &splits, &need);
    if (need > (long)PLM_GEMM_TC_STATIC_SCRATCH_FLOATS) return PLM_ERR_SCRATCH_TOO_SMALL;
    return plm_gemm_tc(x, w, out, out_dtype, T, F, K, ldx, ldw, ldo, g_scratch_ptr[dev], status, stream);
}
