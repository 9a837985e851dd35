// out[T, F] = X[T, K] * W[F, K]^T for few tokens (T <= 64), the shape of a decode
// step: the product is bound by reading W once from HBM, so W takes the 128-row
// side of tcgen05.mma (full tiles), the tokens take 16, 32 or 64 accumulator
// columns, and K is split over the CTAs of a thread-block cluster so that every
// SM streams a share of W.
//
// The K splits' partial sums never go to global memory: every CTA of the cluster
// owns a slice of the tile's rows, each CTA sends the rows of its fp32 partial
// tile straight from tensor memory to their owners' shared memory (stores into
// distributed shared memory), the cluster meets at a barrier, and every CTA sums
// what it received (ascending rank: a fixed order) and writes its slice of the
// result.  Epilogues:
//   EPI_STORE   out = sum                                  (fp32 or bf16)
//   EPI_SWIGLU  W's rows come in tiles of 64 gate rows followed by their 64 up rows;
//               out[t, f] = silu(gate) * up, each rounded to bf16 first
//               (picolm/model_core.c:2182-2193: hb = silu(Wg x) * (Wu x))
//   EPI_RESIDUAL  the product in front of an RMSNorm: the residual add, the norm's weight and
//               the rows' sums of squares in the epilogue (struct Fuse below);
//   SCALE       the product behind it: each token's results times that token's 1/rms.
// The reference's counterpart is its per-row matvec (picolm/tensor.c:839-1419).
//
// Warp roles and pipeline as in gemm_tc.cu; waits are bounded there and here.
// With programmatic dependent launch the weight tiles of the first ring are
// requested before the previous kernel has finished; activations only after.
#include "tc_common.cuh"

using namespace plm_tc;

namespace {

constexpr int EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2;
// ring depth: with the buffer that receives the partial sums (bn x 128 floats), two CTAs of any tile
// width fit one SM (2 x ~105 KB)
__host__ __device__ constexpr int stages_of(int bn) { return bn <= 16 ? 5 : (bn <= 32 ? 4 : 3); }
constexpr int MAX_SPLITS = 8;               // portable cluster size (clusters of 16 were measured: much slower)

__device__ __forceinline__ void st_cluster(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__host__ __device__ constexpr size_t skinny_smem(int bn) {
    return (size_t)stages_of(bn) * (BM * BK * 2 + bn * BK * 2) + (size_t)bn * BM * 4 + 1024 + 256;
}

// A test build only (-DPLM_TEST_STALL, never the library that serves): while the switch is on, the producer
// announces 64 bytes more for every stage than it loads, so no stage ever fills.  Every wait of the kernel
// then runs out: the kernel must record that in the status word, let what it has in flight land, free its
// tensor memory and return.  Nothing faults and nothing is left running.
#ifdef PLM_TEST_STALL
__device__ int plm_stall_switch = 0;
#define PLM_STALL_BYTES (plm_stall_switch ? 64u : 0u)
#else
#define PLM_STALL_BYTES 0u
#endif

constexpr int SS_STRIDE = 64;   // tokens per row of the partial sums of squares that this kernel writes (the most it takes)

// W: [F, K] (P operand, 128 rows per tile), X: [T, K] (Q operand, BN rows).  grid = (F tiles, 1, S),
// cluster = (1, 1, S).  out row stride ldo.  For EPI_SWIGLU, F counts W's rows (gate and up together)
// and out has F/2 columns.
template <int BN, int EPI, typename OutT, bool SCALE>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      OutT* __restrict__ out, int F, int T, int K, long ldo, int kb_per_split, int* __restrict__ status,
                      const Fuse fz) {
    constexpr int STAGES = stages_of(BN);
    constexpr uint32_t W_BYTES = BM * BK * 2, X_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    static_assert(BN * BM * 4 <= STAGES * (W_BYTES + X_BYTES), "the squares must fit the ring");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t w_smem = base, x_smem = base + STAGES * W_BYTES;
    const uint32_t recv_smem = x_smem + STAGES * X_BYTES;              // what the cluster sends here: never the ring,
    const uint32_t bars = recv_smem + BN * BM * 4;                     // which this CTA may still be reading
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tmem_full = bars + 16 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars + 16 * STAGES + 8 - raw));
    // recv[source rank][token][half][row of the slice]: the partial sums of this CTA's rows (half: the
    // gate and the up row of an output column with EPI_SWIGLU)
    const float* recv = reinterpret_cast<const float*>(smem_raw + (recv_smem - raw));
    float* squares = reinterpret_cast<float*>(smem_raw + (base - raw));  // EPI_RESIDUAL, after the main loop:
                                                                         // [BN][rows of this CTA's slice]
    __shared__ int s_abort;
    __shared__ float s_scale[BN];
    __shared__ float s_part[8 * 64];                                   // SCALE: eight partial sums a token

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * BM;
    const uint32_t S = gridDim.z, rank = cluster_rank();
    const int n_kb_total = (K + BK - 1) / BK;
    const int kb_begin = (int)rank * kb_per_split;
    const int kb_end = min(n_kb_total, kb_begin + kb_per_split);
    const int n_kb = max(0, kb_end - kb_begin);

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
    // Shared memory of another CTA may be written only once that CTA runs: a first meeting of the
    // cluster, whose wait every warp does before its own work (warp 0 after it has asked for weights).
    cluster_arrive();
    constexpr int ROWS = EPI == EPI_SWIGLU ? BM / 2 : BM;          // rows that produce an output column
    constexpr int HALVES = BM / ROWS;
    const int slice = ROWS / (int)S;                               // output rows that a CTA of the cluster owns

    if (warp == 0) {
        const int early = n_kb < STAGES ? n_kb : STAGES;
        if (lane == 0) {
            for (int i = 0; i < early; ++i) {                      // weights: nobody in this step writes them
                mbar_expect_tx(full0 + 8 * i, W_BYTES + X_BYTES + PLM_STALL_BYTES);
                tma_load_2d(w_smem + i * W_BYTES, &map_w, full0 + 8 * i, (kb_begin + i) * BK, p0);
            }
        }
        __syncwarp();
        cluster_wait();
        if (lane == 0) {
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(x_smem + i * X_BYTES, &map_x, full0 + 8 * i, (kb_begin + i) * BK, 0);
            int issued = early;
            for (int i = early; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (*(volatile int*)&s_abort) break;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1, status, 1)) { s_abort = 1; break; }
                mbar_expect_tx(full0 + 8 * s, W_BYTES + X_BYTES + PLM_STALL_BYTES);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(w_smem + s * W_BYTES, &map_w, full0 + 8 * s, k, p0);
                tma_load_2d(x_smem + s * X_BYTES, &map_x, full0 + 8 * s, k, 0);
                issued = i + 1;
            }
            if (*(volatile int*)&s_abort)
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr, 0);
        }
    } else if (warp == 1) {
        cluster_wait();
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (*(volatile int*)&s_abort) break;
                if (!mbar_wait(full0 + 8 * s, phase, status, 2)) { s_abort = 1; break; }
                tc_fence_after();
                const uint64_t wd = smem_desc_sw128(w_smem + s * W_BYTES);
                const uint64_t xd = smem_desc_sw128(x_smem + s * X_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_bf16(tmem_base, wd + (uint64_t)(k * UMMA_K * 2 / 16), xd + (uint64_t)(k * UMMA_K * 2 / 16),
                                idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty0 + 8 * s);
            }
            tc_commit(tmem_full);
        }
    } else {
        cluster_wait();
        if (SCALE) {                                       // while the main loop runs: the rows' scale factors
            pdl_wait();
            // The 128 threads share the partial sums: thread (group, j) adds every eighth part of the tokens
            // j, j + 16, ...; then one thread a token adds the eight groups' sums in order.  The order of the
            // additions does not depend on the tile width, so neither does the result.
            const int idx = threadIdx.x - 64, grp = idx >> 4, j = idx & 15;
            for (int t = j; t < BN; t += 16) {
                float ss = 0.f;
                if (t < T)
                    for (int p = grp; p < fz.n_parts; p += 8) ss += fz.scale_parts[(size_t)p * fz.ld_parts + t];
                s_part[grp * 64 + t] = ss;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");             // the four warps of this branch
            if (idx < BN) {
                float ss = 0.f;
#pragma unroll
                for (int g = 0; g < 8; ++g) ss += s_part[g * 64 + idx];
                s_scale[idx] = 1.0f / sqrtf(ss * fz.inv_size + fz.eps);
            }
        }
        // send this CTA's partial tile, row by row, to the CTAs that own the rows
        const int quarter = warp & 3;
        const bool ready = mbar_wait(tmem_full, 0, status, 3);
        if (!ready) s_abort = 1;
        tc_fence_after();
        const int row = quarter * 32 + lane;
        const int orow = row % ROWS, half = row / ROWS;                // output row, and gate or up
        const int owner = orow / slice, pr = orow - owner * slice;
        const uint32_t dst = cluster_map(recv, (uint32_t)owner)
                           + (uint32_t)((((int)rank * BN) * HALVES + half) * slice + pr) * 4u;
        const uint32_t col_stride = (uint32_t)(HALVES * slice) * 4u;
        constexpr int CHUNK = BN >= 32 ? 32 : 16;
#pragma unroll 1
        for (int c = 0; c < BN; c += CHUNK) {
            uint32_t r[32];
            if (ready && n_kb > 0) {
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c;
                if (CHUNK == 32) tc_ld32(taddr, r); else tc_ld16(taddr, r);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK; ++j) r[j] = 0u;              // a CTA without K blocks adds nothing
            }
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) st_cluster(dst + (uint32_t)(c + j) * col_stride, __uint_as_float(r[j]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (*(volatile int*)&s_abort && lane == 0) mbar_wait(tmem_full, 0, nullptr, 0);
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    cluster_sync_all();                                            // everything sent has arrived

    // ---- this CTA sums what it received for its slice of the tile's rows and writes it
    pdl_wait();
    const int items = slice * BN;
    auto received = [&](int c, int half, int pr) {
        float v = 0.f;
#pragma unroll
        for (uint32_t r = 0; r < MAX_SPLITS; ++r)
            if (r < S) v += recv[(((int)r * BN + c) * HALVES + half) * slice + pr];
        return v;
    };
    // The residual epilogue four features at a time where everything is aligned for it (the usual case):
    // 16-byte loads of the partial sums and of the stream, 8-byte loads and stores of the bf16 sides.
    bool residual_done = false;                                    // (any of the wide forms below ran)
    if constexpr (EPI == EPI_RESIDUAL) {
        if (slice % 4 == 0 && ldo % 4 == 0 && fz.ld_xw % 4 == 0 && ((uintptr_t)out & 15) == 0 &&
            ((uintptr_t)fz.xw & 7) == 0 && ((uintptr_t)fz.norm_w & 7) == 0) {
            residual_done = true;
            const int quads = slice / 4;
            for (int it = threadIdx.x; it < quads * BN; it += NUM_THREADS) {
                const int c = it / quads, pr = (it - c * quads) * 4;
                const int t = c, f = p0 + (int)rank * slice + pr;
                float sq[4] = {0.f, 0.f, 0.f, 0.f};
                if (t < T && f < F) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (uint32_t r = 0; r < MAX_SPLITS; ++r)
                        if (r < S) {
                            const float4 p = *reinterpret_cast<const float4*>(&recv[((int)r * BN + c) * slice + pr]);
                            v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
                        }
                    float* xp = reinterpret_cast<float*>(out) + (size_t)t * ldo + f;
                    bf16* wp = fz.xw + (size_t)t * fz.ld_xw + f;
                    if (f + 3 < F) {
                        const float4 x = *reinterpret_cast<const float4*>(xp);
                        const float xn[4] = {x.x + v.x, x.y + v.y, x.z + v.z, x.w + v.w};
                        *reinterpret_cast<float4*>(xp) = make_float4(xn[0], xn[1], xn[2], xn[3]);
                        const uint2 nw = *reinterpret_cast<const uint2*>(fz.norm_w + f);
                        const __nv_bfloat162 n01 = *reinterpret_cast<const __nv_bfloat162*>(&nw.x);
                        const __nv_bfloat162 n23 = *reinterpret_cast<const __nv_bfloat162*>(&nw.y);
                        __nv_bfloat162 o01 = __floats2bfloat162_rn(xn[0] * __low2float(n01), xn[1] * __high2float(n01));
                        __nv_bfloat162 o23 = __floats2bfloat162_rn(xn[2] * __low2float(n23), xn[3] * __high2float(n23));
                        uint2 o;
                        o.x = *reinterpret_cast<uint32_t*>(&o01);
                        o.y = *reinterpret_cast<uint32_t*>(&o23);
                        *reinterpret_cast<uint2*>(wp) = o;
#pragma unroll
                        for (int e = 0; e < 4; ++e) sq[e] = xn[e] * xn[e];
                    } else {
                        const float vv[4] = {v.x, v.y, v.z, v.w};
                        for (int e = 0; e < 4 && f + e < F; ++e) {
                            const float xn = xp[e] + vv[e];
                            xp[e] = xn;
                            wp[e] = __float2bfloat16_rn(xn * __bfloat162float(fz.norm_w[f + e]));
                            sq[e] = xn * xn;
                        }
                    }
                }
                *reinterpret_cast<float4*>(&squares[c * slice + pr]) = make_float4(sq[0], sq[1], sq[2], sq[3]);
            }
        }
    }
    // The same for the store and SwiGLU epilogues with bf16 output: four results, one 8-byte store.
    if constexpr (EPI != EPI_RESIDUAL && sizeof(OutT) == 2) {
        const int n_out = EPI == EPI_SWIGLU ? F / 2 : F;
        const int o0 = (EPI == EPI_SWIGLU ? p0 / 2 : p0) + (int)rank * slice;       // first output column of this CTA
        if (slice % 4 == 0 && ldo % 4 == 0 && n_out % 4 == 0 && ((uintptr_t)out & 7) == 0) {
            residual_done = true;
            const int quads = slice / 4;
            for (int it = threadIdx.x; it < quads * BN; it += NUM_THREADS) {
                const int c = it / quads, pr = (it - c * quads) * 4;
                const int t = c, fo = o0 + pr;
                if (t >= T || fo >= n_out) continue;                                  // n_out % 4 == 0: whole quads only
                float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
#pragma unroll
                for (uint32_t r = 0; r < MAX_SPLITS; ++r)
                    if (r < S) {
                        const float4 p = *reinterpret_cast<const float4*>(&recv[(((int)r * BN + c) * HALVES) * slice + pr]);
                        g.x += p.x; g.y += p.y; g.z += p.z; g.w += p.w;
                        if (EPI == EPI_SWIGLU) {
                            const float4 q = *reinterpret_cast<const float4*>(&recv[(((int)r * BN + c) * HALVES + 1) * slice + pr]);
                            u.x += q.x; u.y += q.y; u.z += q.z; u.w += q.w;
                        }
                    }
                float v[4] = {g.x, g.y, g.z, g.w};
                if (SCALE) {
                    const float sc = s_scale[c];
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] *= sc;
                    u.x *= sc; u.y *= sc; u.z *= sc; u.w *= sc;
                }
                if (EPI == EPI_SWIGLU) {
                    v[0] = swiglu_bf16(v[0], u.x); v[1] = swiglu_bf16(v[1], u.y);
                    v[2] = swiglu_bf16(v[2], u.z); v[3] = swiglu_bf16(v[3], u.w);
                }
                __nv_bfloat162 o01 = __floats2bfloat162_rn(v[0], v[1]), o23 = __floats2bfloat162_rn(v[2], v[3]);
                uint2 o;
                o.x = *reinterpret_cast<uint32_t*>(&o01);
                o.y = *reinterpret_cast<uint32_t*>(&o23);
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + (size_t)t * ldo + fo) = o;
            }
        }
    }
    for (int it = threadIdx.x; it < items && !residual_done; it += NUM_THREADS) {
        const int c = it / slice, pr = it - c * slice;
        const int row = (int)rank * slice + pr;
        const int t = c;
        if (EPI == EPI_RESIDUAL) {
            const int f = p0 + row;
            float sq = 0.f;
            if (t < T && f < F) {
                const float v = received(c, 0, pr);
                const float xn = to_f32(out[(size_t)t * ldo + f]) + v;
                out[(size_t)t * ldo + f] = from_f32<OutT>(xn);
                fz.xw[(size_t)t * fz.ld_xw + f] = __float2bfloat16_rn(xn * __bfloat162float(fz.norm_w[f]));
                sq = xn * xn;
            }
            squares[it] = sq;                                      // [token][row of the slice]
            continue;
        }
        if (t >= T) continue;
        if (EPI == EPI_STORE) {
            const int f = p0 + row;
            if (f >= F) continue;
            float v = received(c, 0, pr);
            if (SCALE) v *= s_scale[c];
            out[(size_t)t * ldo + f] = from_f32<OutT>(v);
        } else {
            const int fo = p0 / 2 + row;
            if (fo >= F / 2) continue;
            float g = received(c, 0, pr), u = received(c, HALVES - 1, pr);
            if (SCALE) { g *= s_scale[c]; u *= s_scale[c]; }
            out[(size_t)t * ldo + fo] = from_f32<OutT>(swiglu_bf16(g, u));
        }
    }
    __syncthreads();                                               // reconverge before the aligned barrier
    if (EPI == EPI_RESIDUAL && threadIdx.x < BN && threadIdx.x < T) {
        float ss = 0.f;
        for (int pr = 0; pr < slice; ++pr) ss += squares[threadIdx.x * slice + pr];
        fz.ss_out[((size_t)blockIdx.x * S + rank) * SS_STRIDE + threadIdx.x] = ss;
    }
    // (no second meeting: after the first nobody touches another CTA's shared memory)
}

template <int BN, int EPI, typename OutT, bool SCALE>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, OutT* out, int F, int T, int K, long ldo, int S, int* status,
           const Fuse& fz, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = skinny_smem(BN);
    auto kern = gemm_tc_skinny_kernel<BN, EPI, OutT, SCALE>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int n_kb = (K + BK - 1) / BK;
    const int per = (n_kb + S - 1) / S;
    return plm_status_of(launch_pdl_cluster(kern, dim3((F + BM - 1) / BM, 1, S), dim3(NUM_THREADS), dim3(1, 1, S), smem, stream,
                                            mw, mx, out, F, T, K, ldo, per, status, fz));
}

// ---- The walk: products with more tiles than two CTAs an SM hold at once (the LM head: 1,002 tiles of 128 rows
// at a vocabulary of 128,256), no split of K, plain store.  A CTA that starts, fills its ring, drains it and
// writes its tile leaves the SM's share of the bandwidth idle at both ends; here two CTAs an SM stay and take the
// tiles blockIdx.x, blockIdx.x + gridDim.x, ... one after another: the ring keeps filling across the tiles'
// boundaries, the accumulator has two places in tensor memory, and the four epilogue warps write tile i (each
// thread one feature's results straight from tensor memory, a warp 32 neighbouring features of one token)
// while the MMAs of tile i + 1 run.  K blocks and their order are those of the kernel above, so are the results.
// (one CTA an SM with a ring twice as deep deals the tiles more evenly and measured 2 % slower: 84.2 against 82.6 us
// for 8 tokens x 128,256 x 2,048)
constexpr int WALK_CTAS_PER_SM = 2;
__host__ __device__ constexpr int walk_stages_of(int bn) {
    return WALK_CTAS_PER_SM == 1 ? (bn <= 16 ? 12 : (bn <= 32 ? 11 : 9)) : (bn <= 16 ? 6 : (bn <= 32 ? 5 : 4));
}
__host__ __device__ constexpr size_t walk_smem(int bn) {
    return (size_t)walk_stages_of(bn) * (BM * BK * 2 + bn * BK * 2) + 1024 + 256;
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, WALK_CTAS_PER_SM)
gemm_tc_skinny_walk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           OutT* __restrict__ out, int F, int T, int K, long ldo, int n_tiles, int* __restrict__ status) {
    constexpr int STAGES = walk_stages_of(BN);
    constexpr uint32_t W_BYTES = BM * BK * 2, X_BYTES = BN * BK * 2;
    constexpr uint32_t ACC_COLS = BN < 32 ? 32 : BN, TMEM_COLS = 2 * ACC_COLS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t w_smem = base, x_smem = base + STAGES * W_BYTES;
    const uint32_t bars = x_smem + STAGES * X_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, acc_full0 = bars + 16 * STAGES, acc_empty0 = acc_full0 + 16,
                   drained = acc_empty0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (drained + 8 - raw));
    __shared__ int s_abort;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + BK - 1) / BK;
    const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total = my_tiles * n_kb;                             // K blocks of all this CTA's tiles, in ring order

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, 128);
        }
        mbar_init(drained, 1);
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
        if (lane == 0) {
            auto tile_row = [&](int g) { return ((int)blockIdx.x + (g / n_kb) * (int)gridDim.x) * BM; };
            const int early = total < STAGES ? total : STAGES;
            for (int g = 0; g < early; ++g) {                      // weights: nobody in this step writes them
                mbar_expect_tx(full0 + 8 * g, W_BYTES + X_BYTES);
                tma_load_2d(w_smem + g * W_BYTES, &map_w, full0 + 8 * g, (g % n_kb) * BK, tile_row(g));
            }
            pdl_wait();                                            // the activations come from the kernel before
            for (int g = 0; g < early; ++g)
                tma_load_2d(x_smem + g * X_BYTES, &map_x, full0 + 8 * g, (g % n_kb) * BK, 0);
            int issued = early;
            for (int g = early; g < total; ++g) {
                const int s = g % STAGES;
                if (*(volatile int*)&s_abort) break;
                if (!mbar_wait(empty0 + 8 * s, ((g / STAGES) & 1) ^ 1, status, 1)) { s_abort = 1; break; }
                mbar_expect_tx(full0 + 8 * s, W_BYTES + X_BYTES);
                const int k = (g % n_kb) * BK;
                tma_load_2d(w_smem + s * W_BYTES, &map_w, full0 + 8 * s, k, tile_row(g));
                tma_load_2d(x_smem + s * X_BYTES, &map_x, full0 + 8 * s, k, 0);
                issued = g + 1;
            }
            if (*(volatile int*)&s_abort)
                for (int g = max(0, issued - STAGES); g < issued; ++g)
                    mbar_wait(full0 + 8 * (g % STAGES), (g / STAGES) & 1, nullptr, 0);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            bool ok = true;
            int g = 0;
            for (int it = 0; it < my_tiles && ok; ++it) {
                const int a = it & 1;                              // the accumulator's place; free once tile it - 2 is written
                if (!mbar_wait(acc_empty0 + 8 * a, ((it >> 1) & 1) ^ 1, status, 2)) { ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < n_kb; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    if (!mbar_wait(full0 + 8 * s, (g / STAGES) & 1, status, 2)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t wd = smem_desc_sw128(w_smem + s * W_BYTES);
                    const uint64_t xd = smem_desc_sw128(x_smem + s * X_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_bf16(tmem_base + a * ACC_COLS, wd + (uint64_t)(k * UMMA_K * 2 / 16),
                                    xd + (uint64_t)(k * UMMA_K * 2 / 16), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);
                }
                if (ok) tc_commit(acc_full0 + 8 * a);
            }
            if (!ok) {                                             // nothing may be in flight when the tensor memory goes
                s_abort = 1;
                tc_commit(drained);
                mbar_wait(drained, 0, nullptr, 0);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        constexpr int CHUNK = BN >= 32 ? 32 : 16;
        pdl_wait();                                                // whoever read the last step's results is done
        for (int it = 0; it < my_tiles; ++it) {
            const int a = it & 1;
            if (*(volatile int*)&s_abort) break;
            if (!mbar_wait(acc_full0 + 8 * a, (it >> 1) & 1, status, 3)) { s_abort = 1; break; }
            tc_fence_after();
            const int f = ((int)blockIdx.x + it * (int)gridDim.x) * BM + row;
#pragma unroll 1
            for (int c = 0; c < BN; c += CHUNK) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * ACC_COLS + c);
                if (CHUNK == 32) tc_ld32(taddr, r); else tc_ld16(taddr, r);
                tc_wait_ld();
                if (f < F) {
#pragma unroll
                    for (int j = 0; j < CHUNK; ++j)
                        if (c + j < T) out[(size_t)(c + j) * ldo + f] = from_f32<OutT>(__uint_as_float(r[j]));
                }
            }
            tc_fence_before();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * a) : "memory");
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

template <int BN, typename OutT>
int launch_walk(const CUtensorMap& mw, const CUtensorMap& mx, OutT* out, int F, int T, int K, long ldo, int* status,
                cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = walk_smem(BN);
    auto kern = gemm_tc_skinny_walk_kernel<BN, OutT>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int n_tiles = (F + BM - 1) / BM;
    return plm_status_of(launch_pdl(kern, dim3(WALK_CTAS_PER_SM * PLM_SM_COUNT), dim3(NUM_THREADS), smem, stream, mw, mx, out, F, T, K,
                                    ldo, n_tiles, status));
}

template <typename OutT>
int dispatch_walk(int bn, const CUtensorMap& mw, const CUtensorMap& mx, OutT* out, int F, int T, int K, long ldo,
                  int* status, cudaStream_t stream) {
    if (bn == 16) return launch_walk<16, OutT>(mw, mx, out, F, T, K, ldo, status, stream);
    if (bn == 32) return launch_walk<32, OutT>(mw, mx, out, F, T, K, ldo, status, stream);
    return launch_walk<64, OutT>(mw, mx, out, F, T, K, ldo, status, stream);
}

// Whether a plain product of (F, K) walks: more tiles than two CTAs an SM hold, so K is not split either.
inline bool walks(int F) { return (F + BM - 1) / BM > 2 * PLM_SM_COUNT; }

template <int EPI, typename OutT, bool SCALE = false>
int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, OutT* out, int F, int T, int K, long ldo, int S,
                int* status, cudaStream_t stream, const Fuse& fz = Fuse{}) {
    if (bn == 16) return launch<16, EPI, OutT, SCALE>(mw, mx, out, F, T, K, ldo, S, status, fz, stream);
    if (bn == 32) return launch<32, EPI, OutT, SCALE>(mw, mx, out, F, T, K, ldo, S, status, fz, stream);
    return launch<64, EPI, OutT, SCALE>(mw, mx, out, F, T, K, ldo, S, status, fz, stream);
}

}  // namespace

#ifdef PLM_TEST_STALL
extern "C" int plm_test_stall(int on, cudaStream_t stream) {
    return plm_status_of(cudaMemcpyToSymbolAsync(plm_stall_switch, &on, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
}
#endif

// How many CTAs share a tile's K range: the largest power of two (at most 8) that keeps the grid
// within one wave of two CTAs per SM and leaves every CTA at least two K blocks.  Fixed by (F, K).
extern "C" int plm_gemm_tc_skinny_splits(int F, int K) {
    const int tiles = (F + BM - 1) / BM;
    const int n_kb = (K + BK - 1) / BK;
    int S = MAX_SPLITS;
    while (S > 1 && (tiles * S > 2 * PLM_SM_COUNT || n_kb < 2 * S)) S >>= 1;
    return S;
}

// out[T, F'] = epilogue(x[T, K] * w[F, K]^T), T <= 64, bf16 operands.  epilogue 0: F' = F, out is
// float32 (out_dtype 0) or bfloat16 (1).  epilogue 1 (SwiGLU): w holds tiles of 64 gate rows followed
// by their 64 up rows (F a multiple of 128), F' = F / 2, out is bfloat16.
extern "C" int plm_gemm_tc_skinny(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                  int K, long ldx, long ldw, long ldo, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (T > 64) return PLM_ERR_UNSUPPORTED;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && (F % 128 || out_dtype != PLM_BF16)) return PLM_ERR_SHAPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) return PLM_ERR_UNSUPPORTED;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    const int S = plm_gemm_tc_skinny_splits(F, K);
    CUtensorMap mw, mx;
    int rc;
    if ((rc = make_map(&mw, w, F, K, ldw, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mx, x, T, K, ldx, bn)) != PLM_OK) return rc;
    if (epilogue == EPI_SWIGLU)
        return dispatch_bn<EPI_SWIGLU, bf16>(bn, mw, mx, (bf16*)out, F, T, K, ldo, S, status, stream);
    if (walks(F) && out_dtype == PLM_F32) return dispatch_walk<float>(bn, mw, mx, (float*)out, F, T, K, ldo, status, stream);
    if (walks(F) && out_dtype == PLM_BF16) return dispatch_walk<bf16>(bn, mw, mx, (bf16*)out, F, T, K, ldo, status, stream);
    if (out_dtype == PLM_F32) return dispatch_bn<EPI_STORE, float>(bn, mw, mx, (float*)out, F, T, K, ldo, S, status, stream);
    if (out_dtype == PLM_BF16) return dispatch_bn<EPI_STORE, bf16>(bn, mw, mx, (bf16*)out, F, T, K, ldo, S, status, stream);
    return PLM_ERR_DTYPE;
}

// Rows of partial sums of squares that plm_gemm_tc_skinny_residual writes for (F, K): one per (tile,
// cluster rank), each of 64 floats.
extern "C" int plm_gemm_tc_skinny_residual_parts(int F, int K) {
    return ((F + BM - 1) / BM) * plm_gemm_tc_skinny_splits(F, K);
}

// The product in front of an RMSNorm: resid[T, F] += x[T, K] * w[F, K]^T in place (fp32), xw[T, F] =
// bf16(new resid * norm_w), ss_out[parts, 64] = partial sums of squares of the new rows (see Fuse).
extern "C" int plm_gemm_tc_skinny_residual(const void* x, const void* w, float* resid, const void* norm_w, void* xw,
                                           float* ss_out, int T, int F, int K, long ldx, long ldw, long ld_resid,
                                           long ld_xw, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (T > 64) return PLM_ERR_UNSUPPORTED;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if (!resid || !norm_w || !xw || !ss_out) return PLM_ERR_SHAPE;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    const int S = plm_gemm_tc_skinny_splits(F, K);
    CUtensorMap mw, mx;
    int rc;
    if ((rc = make_map(&mw, w, F, K, ldw, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mx, x, T, K, ldx, bn)) != PLM_OK) return rc;
    Fuse fz = {};
    fz.norm_w = (const bf16*)norm_w;
    fz.xw = (bf16*)xw;
    fz.ld_xw = ld_xw;
    fz.ss_out = ss_out;
    return dispatch_bn<EPI_RESIDUAL, float>(bn, mw, mx, resid, F, T, K, ld_resid, S, status, stream, fz);
}

// The product behind an RMSNorm whose weight is already in x (see Fuse): like plm_gemm_tc_skinny with
// bfloat16 output, token t's results scaled by 1 / sqrt(sum_p scale_parts[p, t] / size + eps).
extern "C" int plm_gemm_tc_skinny_scaled(const void* x, const void* w, void* out, int epilogue, int T, int F, int K,
                                         long ldx, long ldw, long ldo, const float* scale_parts, int n_parts,
                                         int ld_parts, int size, float eps, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (T > 64) return PLM_ERR_UNSUPPORTED;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && F % 128) return PLM_ERR_SHAPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU) return PLM_ERR_UNSUPPORTED;
    if (!scale_parts || n_parts <= 0 || size <= 0 || ld_parts < T) return PLM_ERR_SHAPE;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    const int S = plm_gemm_tc_skinny_splits(F, K);
    CUtensorMap mw, mx;
    int rc;
    if ((rc = make_map(&mw, w, F, K, ldw, BM)) != PLM_OK) return rc;
    if ((rc = make_map(&mx, x, T, K, ldx, bn)) != PLM_OK) return rc;
    Fuse fz = {};
    fz.scale_parts = scale_parts;
    fz.n_parts = n_parts;
    fz.ld_parts = ld_parts;
    fz.inv_size = 1.0f / (float)size;
    fz.eps = eps;
    if (epilogue == EPI_SWIGLU)
        return dispatch_bn<EPI_SWIGLU, bf16, true>(bn, mw, mx, (bf16*)out, F, T, K, ldo, S, status, stream, fz);
    return dispatch_bn<EPI_STORE, bf16, true>(bn, mw, mx, (bf16*)out, F, T, K, ldo, S, status, stream, fz);
}
