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
//   EPI_RESIDUAL out += product, out being the fp32 residual stream (x = x + delta,
//               picolm/model_core.c:3120 and 3201).  A thread of the epilogue holds one token's row of
//               the accumulator, and rows of the stream lie far apart: each warp turns its 32 x 32 piece
//               over in shared memory, so that a quarter of a warp reads, adds to and writes 128
//               consecutive bytes of one row.
// Warp 0 loads (TMA), warp 1 issues the MMAs and owns the tensor memory, warps 2..5 are the
// epilogue.  Waits on mbarriers are bounded; a wait that runs out records where in `status`
// and the CTA drains and leaves.
//
// K splits (single CTAs, store epilogue): where a problem has fewer tiles than SMs (prompts of a few
// hundred tokens), every tile's K range is cut into `k_splits` parts that are units of work of their own;
// each writes its fp32 partial tile to its own slice of a scratch buffer, and a second kernel adds the
// slices up in order and converts.
//
// PAIR: two CTAs of a cluster (two SMs) work on one tile of 256 tokens x 256 features with
// tcgen05.mma.cta_group::2.  Each CTA loads its 128 token rows and HALF of the weight tile (128
// features), the tensor cores of both SMs read both halves, and each CTA's tensor memory receives
// its own 128 rows of the result.  A 128 x 256 tile is bound by what an SM has to bring in from L2
// per MMA cycle (48 KB per K block of 64); the pair brings in 32 KB each for the same work.  The
// CTA of rank 0 issues all MMAs: both CTAs' loads signal ITS "full" barriers (expect-tx set there),
// its commits arrive at the "empty" and "accumulator full" barriers of both CTAs (commit with
// multicast), and both CTAs' epilogues arrive at ITS "accumulator empty" barriers.  No TMA load
// uses multicast.
#include "tc_common.cuh"

using namespace plm_tc;

namespace {

constexpr int EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2;
constexpr int TURN_LD = 36;                                  // floats per row of a warp's 32 x 32 piece: 16-byte rows, no bank conflicts
constexpr size_t TURN_BYTES = 4 * 32 * TURN_LD * 4;          // for the four epilogue warps

__host__ __device__ constexpr int stages_of(int bn) { return bn >= 256 ? 4 : 6; }
__host__ __device__ constexpr size_t wide_smem(int bn, int epi = EPI_STORE) {
    return (size_t)stages_of(bn) * (BM * BK * 2 + bn * BK * 2) + 1024 + 256 + (epi == EPI_RESIDUAL ? TURN_BYTES : 0);
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// --- the forms for a pair of CTAs (cta_group::2); `bar` of the first three is a shared::cluster address
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {           // arrives at `bar` in both CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D fp32, A and B bf16, both K-major, M = 256 over the pair, N = n
__host__ __device__ constexpr uint32_t instr_desc_bf16_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__host__ __device__ constexpr int pair_stages() { return 6; }
__host__ __device__ constexpr size_t pair_smem(int epi = EPI_STORE) {
    return (size_t)pair_stages() * (BM * BK * 2 + 128 * BK * 2) + 1024 + 256 + (epi == EPI_RESIDUAL ? TURN_BYTES : 0);
}

template <int BN, int EPI, typename OutT, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    OutT* __restrict__ out, int T, int F, int K, long ldo, int m_tiles, int n_tiles,
                    int* __restrict__ status, int k_splits, int kb_per_split, size_t split_stride) {
    static_assert(!PAIR || BN == 256, "the pair works on tiles of 256 x 256");
    constexpr int STAGES = PAIR ? pair_stages() : stages_of(BN);
    constexpr int W_ROWS = PAIR ? BN / 2 : BN;                           // weight rows that this CTA loads per K block
    constexpr uint32_t X_BYTES = BM * BK * 2, W_BYTES = W_ROWS * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;                               // two accumulators
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t x_smem = base, w_smem = base + STAGES * X_BYTES;
    const uint32_t bars = w_smem + STAGES * W_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, acc_full0 = bars + 16 * STAGES,
                   acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (acc_empty0 + 16 - raw));
    float* turn_base = reinterpret_cast<float*>(smem_raw + (bars + 256 - raw));    // EPI_RESIDUAL only
    __shared__ int s_abort;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + BK - 1) / BK;
    const int n_tiles_mn = m_tiles * n_tiles;                            // PAIR: tiles of 256 tokens
    const int n_tiles_total = n_tiles_mn * k_splits;                     // units of work: (tile, part of K)
    const uint32_t rank = PAIR ? cluster_rank() : 0u;                    // rank 0 of a pair issues the MMAs
    const int first_tile = PAIR ? blockIdx.x / 2 : blockIdx.x, tile_step = PAIR ? gridDim.x / 2 : gridDim.x;
    constexpr int TILE_M = PAIR ? 2 * BM : BM;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, PAIR ? 256 : 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {                                                      // by the same warp of both CTAs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();                                        // both CTAs' barriers exist before either is signalled
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool waited = false;
            int it = 0;                                                  // K blocks issued so far, over all tiles
            bool ok = true;
            for (int unit = first_tile; unit < n_tiles_total && ok; unit += tile_step) {
                const int tile = unit % n_tiles_mn, ks = unit / n_tiles_mn;
                const int kb_begin = ks * kb_per_split, kb_end = min(n_kb, kb_begin + kb_per_split);
                const int m0 = (tile % m_tiles) * TILE_M + (int)rank * BM, f0 = (tile / m_tiles) * BN + (int)rank * W_ROWS;
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, status, 1)) { s_abort = 1; ok = false; break; }
                    if (PAIR) {
                        // both CTAs' tiles count at the "full" barrier of rank 0, which expects them all
                        const uint32_t full = cluster_map_addr(full0 + 8 * s, 0);
                        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * (X_BYTES + W_BYTES));
                        tma_load_2d_pair(w_smem + s * W_BYTES, &map_w, full, kb * BK, f0);
                        if (!waited) { pdl_wait(); waited = true; }
                        tma_load_2d_pair(x_smem + s * X_BYTES, &map_x, full, kb * BK, m0);
                    } else {
                        mbar_expect_tx(full0 + 8 * s, X_BYTES + W_BYTES);
                        // weights are written by no kernel of the step: they may be requested at once
                        tma_load_2d(w_smem + s * W_BYTES, &map_w, full0 + 8 * s, kb * BK, f0);
                        if (!waited) { pdl_wait(); waited = true; }     // activations come from the kernel before
                        tma_load_2d(x_smem + s * X_BYTES, &map_x, full0 + 8 * s, kb * BK, m0);
                    }
                }
            }
            if (*(volatile int*)&s_abort && (!PAIR || rank == 0))
                for (int i = max(0, it - STAGES); i < it; ++i)
                    mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr, 0);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = PAIR ? instr_desc_bf16_pair(BN) : instr_desc_bf16(BN);
            int it = 0, j = 0;
            bool ok = true;
            for (int unit = first_tile; unit < n_tiles_total && ok; unit += tile_step, ++j) {
                const int acc = j & 1;
                const int ks = unit / n_tiles_mn;
                const int kb_begin = ks * kb_per_split, kb_end = min(n_kb, kb_begin + kb_per_split);
                // the epilogue must have read this accumulator's previous tile out
                if (!mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, status, 2)) { s_abort = 1; ok = false; break; }
                tc_fence_after();
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, status, 2)) { s_abort = 1; ok = false; break; }
                    tc_fence_after();
                    const uint64_t xd = smem_desc_sw128(x_smem + s * X_BYTES);
                    const uint64_t wd = smem_desc_sw128(w_smem + s * W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        if (PAIR)
                            tc_mma_bf16_pair(tmem_base + acc * BN, xd + (uint64_t)(k * UMMA_K * 2 / 16),
                                             wd + (uint64_t)(k * UMMA_K * 2 / 16), idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                        else
                            tc_mma_bf16(tmem_base + acc * BN, xd + (uint64_t)(k * UMMA_K * 2 / 16),
                                        wd + (uint64_t)(k * UMMA_K * 2 / 16), idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                    }
                    if (PAIR) tc_commit_pair(empty0 + 8 * s); else tc_commit(empty0 + 8 * s);
                }
                if (PAIR) tc_commit_pair(acc_full0 + 8 * acc); else tc_commit(acc_full0 + 8 * acc);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        pdl_wait();                                                      // the output may still be in use by an earlier kernel
        int j = 0;
        bool ok = true;
        for (int unit = first_tile; unit < n_tiles_total && ok; unit += tile_step, ++j) {
            const int acc = j & 1;
            const int tile = unit % n_tiles_mn, ks = unit / n_tiles_mn;
            const int m0 = (tile % m_tiles) * TILE_M + (int)rank * BM, f0 = (tile / m_tiles) * BN;
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
            } else if (EPI == EPI_RESIDUAL) {
                float* turn = turn_base + quarter * 32 * TURN_LD;
                const int row0 = m0 + quarter * 32;                      // this warp's 32 token rows
                const int sub = lane >> 3, col = (lane & 7) * 4;         // pass p: row 4 p + sub, four columns from col
                float* outf = reinterpret_cast<float*>(out);
                const bool aligned = (ldo % 4 == 0) && ((uintptr_t)outf % 16 == 0);
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (f0 + c >= F) break;
                    const bool vec = aligned && (f0 + c + 32 <= F);
                    float4 old[8];
                    if (vec) {
#pragma unroll
                        for (int p = 0; p < 8; ++p) {
                            const int row = row0 + 4 * p + sub;
                            old[p] = row < T ? *reinterpret_cast<const float4*>(outf + (size_t)row * ldo + f0 + c + col)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                    uint32_t r[32];
                    tc_ld32(tacc + c, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4*>(turn + lane * TURN_LD + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
                    __syncwarp();
#pragma unroll
                    for (int p = 0; p < 8; ++p) {
                        const int row = row0 + 4 * p + sub;
                        const float4 d = *reinterpret_cast<const float4*>(turn + (4 * p + sub) * TURN_LD + col);
                        if (row >= T) continue;
                        float* dst = outf + (size_t)row * ldo + f0 + c + col;
                        if (vec) {
                            *reinterpret_cast<float4*>(dst) = make_float4(old[p].x + d.x, old[p].y + d.y, old[p].z + d.z, old[p].w + d.w);
                        } else {
                            const float dd[4] = {d.x, d.y, d.z, d.w};
                            for (int i = 0; i < 4; ++i)
                                if (f0 + c + col + i < F) dst[i] += dd[i];
                        }
                    }
                    __syncwarp();                                        // the piece is read before the next one overwrites it
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    if (f0 + c >= F) break;
                    uint32_t r[32];
                    tc_ld32(tacc + c, r);
                    tc_wait_ld();
                    if (t < T) {
                        OutT* rowp = out + (size_t)ks * split_stride + (size_t)t * ldo + f0 + c;
                        const bool vec = (f0 + c + 32 <= F) && ((((size_t)ks * split_stride + (size_t)t * ldo + f0 + c) * sizeof(OutT)) % 16 == 0);
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
            // this accumulator may be overwritten (a pair: says so to rank 0, which issues the MMAs)
            if (PAIR) mbar_arrive_cluster(cluster_map_addr(acc_empty0 + 8 * acc, 0)); else mbar_arrive(acc_empty0 + 8 * acc);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();          // the other CTA's MMAs read this CTA's tiles and write its tensor memory
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = PLM_SM_COUNT;
    }
    return n;
}

template <int EPI, typename OutT>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, OutT* out, int T, int F, int K, long ldo, int* status,
                cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = pair_smem(EPI);
    auto kern = gemm_tc_wide_kernel<256, EPI, OutT, true>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = (T + 2 * BM - 1) / (2 * BM), n_tiles = (F + 255) / 256;
    int pairs = sm_count() / 2;
    if (m_tiles * n_tiles < pairs) pairs = m_tiles * n_tiles;
    return plm_status_of(launch_pdl_cluster(kern, dim3(2 * pairs), dim3(NUM_THREADS), dim3(2, 1, 1), smem, stream, mx, mw,
                                            out, T, F, K, ldo, m_tiles, n_tiles, status, 1, (K + BK - 1) / BK, (size_t)0));
}

template <int BN, int EPI, typename OutT>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, OutT* out, int T, int F, int K, long ldo, int* status,
           cudaStream_t stream, int k_splits = 1, int kb_per_split = 0, size_t split_stride = 0) {
    static bool configured = false;
    constexpr size_t smem = wide_smem(BN, EPI);
    auto kern = gemm_tc_wide_kernel<BN, EPI, OutT, false>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = (T + BM - 1) / BM, n_tiles = (F + BN - 1) / BN;
    const int units = m_tiles * n_tiles * k_splits;
    const int ctas = units < sm_count() ? units : sm_count();
    if (kb_per_split <= 0) kb_per_split = (K + BK - 1) / BK;
    return plm_status_of(launch_pdl(kern, dim3(ctas), dim3(NUM_THREADS), smem, stream, mx, mw, out, T, F, K, ldo, m_tiles,
                                    n_tiles, status, k_splits, kb_per_split, split_stride));
}

// out[i] = sum over the K splits of scratch[s * stride + i], in order; four at a time.
template <typename OutT>
__global__ void reduce_splits_kernel(const float* __restrict__ scratch, OutT* __restrict__ out, int k_splits, size_t n4,
                                     size_t stride) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 a = *reinterpret_cast<const float4*>(scratch + 4 * i);
        for (int s = 1; s < k_splits; ++s) {
            const float4 b = *reinterpret_cast<const float4*>(scratch + (size_t)s * stride + 4 * i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (sizeof(OutT) == 4) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + 4 * i) = a;
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + 4 * i) = o;
        }
    }
}

// Tile width and K splits of the single-CTA form for (T, F, K); see plm_gemm_tc_wide.
void wide_plan(int T, int F, int K, int* bn_out, int* k_splits_out, int* kb_per_out) {
    int bn = 128;
    const long m_tiles = (T + BM - 1) / BM, sms = sm_count();
    if (F >= 2048 && T >= 256) {
        const long wide = (m_tiles * ((F + 255) / 256) + sms - 1) / sms, narrow = (m_tiles * ((F + 127) / 128) + sms - 1) / sms;
        bn = 0.8 * (double)narrow < (double)wide ? 128 : 256;
    }
    // K splits where the tiles leave at least half of the SMs without work and K is long enough to cut
    const long tiles = m_tiles * ((F + bn - 1) / bn);
    const int n_kb = (K + BK - 1) / BK;
    int splits = 1;
    if (tiles * 2 <= sms && F % 4 == 0) {
        splits = (int)(sms / tiles);
        if (splits > 8) splits = 8;
        if (splits > n_kb / 4) splits = n_kb / 4;
        if (splits < 1) splits = 1;
    }
    const int per = (n_kb + splits - 1) / splits;
    *bn_out = bn;
    *kb_per_out = per;
    *k_splits_out = (n_kb + per - 1) / per;                                // no part of K is empty
}

}  // namespace

// Into how many parts plm_gemm_tc_wide cuts K for (T, F, K) with the store epilogue: it needs that many
// slices of T * F floats of scratch memory if the answer is more than 1.
extern "C" int plm_gemm_tc_wide_splits(int T, int F, int K) {
    int bn, splits, per;
    wide_plan(T, F, K, &bn, &splits, &per);
    return splits;
}

// out[T, F'] = epilogue(x[T, K] * w[F, K]^T), T > 64, bf16 operands that TMA can address (K and the
// leading dimensions multiples of 8, pointers 16-byte aligned).  epilogue 0: F' = F, out float32
// (out_dtype 0) or bfloat16 (1).  epilogue 1 (SwiGLU): w holds tiles of 64 gate rows followed by their
// 64 up rows (F a multiple of 128), F' = F / 2, out bfloat16.  `scratch`: plm_gemm_tc_wide_splits(T, F, K) slices
// of T * F floats where that is more than 1 (else unused; without it K is not cut).
extern "C" int plm_gemm_tc_wide_scratch(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                        int K, long ldx, long ldw, long ldo, float* scratch, int* status,
                                        cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && (F % 128 || out_dtype != PLM_BF16)) return PLM_ERR_SHAPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) return PLM_ERR_UNSUPPORTED;
    // Tile width: 256 columns feed the tensor cores best (a 128-column tile takes 0.8 of a 256-column tile's
    // time for half the work), but the CTAs walk whole tiles: where the narrow tiles need no more rounds over
    // the SMs than the wide ones (prompts of a few hundred tokens), they finish earlier.
    int bn, k_splits, kb_per;
    wide_plan(T, F, K, &bn, &k_splits, &kb_per);
    CUtensorMap mx, mw;
    int rc;
    if ((rc = make_map(&mx, x, T, K, ldx, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mw, w, F, K, ldw, bn)) != PLM_OK) return rc;
    if (epilogue == EPI_SWIGLU) {
        if (bn == 256) return launch<256, EPI_SWIGLU, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
        return launch<128, EPI_SWIGLU, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
    }
    if (out_dtype != PLM_F32 && out_dtype != PLM_BF16) return PLM_ERR_DTYPE;
    if (k_splits > 1 && scratch && ldo == F && (((uintptr_t)scratch | (uintptr_t)out) & 15) == 0) {
        // the parts of K as units of work of their own, each into its slice of the scratch; then the sum
        const size_t stride = (size_t)T * F;
        rc = bn == 256 ? launch<256, EPI_STORE, float>(mx, mw, scratch, T, F, K, F, status, stream, k_splits, kb_per, stride)
                       : launch<128, EPI_STORE, float>(mx, mw, scratch, T, F, K, F, status, stream, k_splits, kb_per, stride);
        if (rc != PLM_OK) return rc;
        const size_t n4 = stride / 4;
        const int blocks = (int)((n4 + 255) / 256 < (size_t)(8 * sm_count()) ? (n4 + 255) / 256 : (size_t)(8 * sm_count()));
        if (out_dtype == PLM_F32)
            return plm_status_of(launch_pdl(reduce_splits_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                                            (const float*)scratch, (float*)out, k_splits, n4, stride));
        return plm_status_of(launch_pdl(reduce_splits_kernel<bf16>, dim3(blocks), dim3(256), 0, stream,
                                        (const float*)scratch, (bf16*)out, k_splits, n4, stride));
    }
    if (out_dtype == PLM_F32) {
        if (bn == 256) return launch<256, EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
        return launch<128, EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
    }
    if (bn == 256) return launch<256, EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
    return launch<128, EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
}

// The same without scratch memory (K is never cut).
extern "C" int plm_gemm_tc_wide(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                int K, long ldx, long ldw, long ldo, int* status, cudaStream_t stream) {
    return plm_gemm_tc_wide_scratch(x, w, out, out_dtype, epilogue, T, F, K, ldx, ldw, ldo, nullptr, status, stream);
}

// The same product by pairs of CTAs (tcgen05.mma.cta_group::2, tiles of 256 tokens x 256 features; see
// PAIR at the top).  For prompts of at least 256 tokens and at least 256 features.
extern "C" int plm_gemm_tc_pair(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                int K, long ldx, long ldw, long ldo, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && (F % 128 || out_dtype != PLM_BF16)) return PLM_ERR_SHAPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) return PLM_ERR_UNSUPPORTED;
    CUtensorMap mx, mw;
    int rc;
    if ((rc = make_map(&mx, x, T, K, ldx, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mw, w, F, K, ldw, 128)) != PLM_OK) return rc;
    if (epilogue == EPI_SWIGLU) return launch_pair<EPI_SWIGLU, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
    if (out_dtype == PLM_F32) return launch_pair<EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
    if (out_dtype == PLM_BF16) return launch_pair<EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
    return PLM_ERR_DTYPE;
}

// resid[T, F] += x[T, K] * w[F, K]^T in place, resid in float32 (the residual stream), T > 64; operands as for
// plm_gemm_tc_wide.  `pair` != 0: by pairs of CTAs (for at least 256 tokens and 256 features).  K is not cut.
extern "C" int plm_gemm_tc_wide_residual(const void* x, const void* w, float* resid, int T, int F, int K, long ldx,
                                         long ldw, long ldr, int pair, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if ((uintptr_t)resid % 4) return PLM_ERR_ALIGN;
    CUtensorMap mx, mw;
    int rc;
    if ((rc = make_map(&mx, x, T, K, ldx, BM)) != PLM_OK) return rc;
    if (pair) {
        if ((rc = make_map(&mw, w, F, K, ldw, 128)) != PLM_OK) return rc;
        return launch_pair<EPI_RESIDUAL, float>(mx, mw, resid, T, F, K, ldr, status, stream);
    }
    int bn, k_splits, kb_per;
    wide_plan(T, F, K, &bn, &k_splits, &kb_per);
    if ((rc = make_map(&mw, w, F, K, ldw, bn)) != PLM_OK) return rc;
    if (bn == 256) return launch<256, EPI_RESIDUAL, float>(mx, mw, resid, T, F, K, ldr, status, stream);
    return launch<128, EPI_RESIDUAL, float>(mx, mw, resid, T, F, K, ldr, status, stream);
}
