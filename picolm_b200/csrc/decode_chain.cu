// A chain of decode-shaped products in ONE persistent kernel: up to four products of few tokens
// (T <= 64) that feed one another, each with the epilogue that the step needs between them,
//
//   RESIDUAL  x[T, N] += a . W^T in place (fp32 stream); xw = bf16(x * norm_w); per-token partial
//             sums of squares of the new x                (picolm/model_core.c:2149-2160, :2204)
//   SWIGLU    h = silu(g r) * (u r), (g, u) = a . W^T with W's rows in tiles of 64 gate rows and
//             their 64 up rows, r = the token's 1/rms from those sums   (picolm/model_core.c:2182-2193)
//   SCALED    out = bf16((a . W^T) r)                      (the projection behind a norm)
//   PLAIN     out = a . W^T in fp32
//
// which is a Llama layer's output projection, feed-forward and the next layer's query/key/value
// projection when the phases are RESIDUAL, SWIGLU, RESIDUAL, SCALED.  Launched one after another,
// each of these products pays a few microseconds that do not stream weights (the kernel's start,
// its first activation tile, the exchange of partial sums, its epilogue, the wait of the next kernel
// for its end); a decode step is bound by reading the weights, so those microseconds are a third of
// it.  Here one CTA per SM lives through the whole chain:
//
//   * every product's weight blocks (128 rows x 64 of K) are dealt out evenly over the CTAs in
//     (tile, K block) order, so every SM streams the same number of bytes whatever the shape;
//   * a producer thread asks for its CTA's blocks of ALL phases through one ring of shared memory
//     (TMA), running ahead of the phase the others are in: weights depend on nothing, so the ring
//     keeps filling while partial sums are exchanged and epilogues run, and HBM never idles;
//   * the activation tile of a block is asked for once its phase's input exists;
//   * one thread issues tcgen05.mma into one of two accumulators in tensor memory; four warps
//     read finished accumulators back and write them as fp32 partial sums to scratch memory;
//   * all CTAs meet at a counter in global memory, then each CTA sums the partial sums of its share
//     of the product's columns in a fixed order (so the result does not depend on how fast any
//     CTA was), applies the epilogue and writes the phase's output; they meet again, and the next
//     phase's activation tiles may be asked for.
//
// Every wait is bounded (mbarriers and the counter alike): when a bound is hit the CTA records it in
// the status word, lets what it has in flight land, frees its tensor memory and returns; the other
// CTAs see the status word at their next meeting and return too.  The meeting counter is put back
// to zero by the last CTA that leaves, whatever happened.
#include "tc_common.cuh"

using namespace plm_tc;

namespace {

constexpr int MAX_PHASES = 4;
enum { KIND_RESIDUAL = 0, KIND_SWIGLU = 1, KIND_SCALED = 2, KIND_PLAIN = 3 };
constexpr int SS_LD = 64;                   // floats per row of a sums-of-squares table (one row per CTA)
constexpr int MAX_SHARE = 4096;             // (tokens x columns) of a RESIDUAL phase that one CTA sums: 64 x 64
constexpr uint32_t SPIN_LIMIT = 1u << 24;   // polls of the meeting counter before giving up

struct Phase {
    CUtensorMap map_w;                      // [N, K] bf16, boxes of 128 x 64
    CUtensorMap map_a;                      // [T, K] bf16, boxes of BN x 64 (rows beyond T read as zeros)
    int kind, N, K, n_tiles, n_kb, slots;
    long long total;                        // n_tiles * n_kb
    void* out;                              // RESIDUAL: xw bf16; SWIGLU, SCALED: bf16; PLAIN: fp32
    long long ldo;
    float* resid;                           // RESIDUAL: the stream, [T, ld_resid]
    long long ld_resid;
    const bf16* norm_w;                     // RESIDUAL: [N]
    float* ss_out;                          // RESIDUAL: [CTAs, SS_LD], column t for token t
    const float* ss_in;                     // SWIGLU, SCALED: the table a RESIDUAL phase wrote
    float inv_size, eps;
};

struct Chain {
    Phase ph[MAX_PHASES];
    int n_phases, T;
    float* partial;                         // scratch: [tile][slot][BN tokens][128 rows] fp32, sized for the largest phase
    unsigned int* sync;                     // [0]: the meeting counter, [1]: CTAs that have left
    int* status;
};

__host__ __device__ inline long long first_block(long long total, int cta, int n_ctas) {
    return total * cta / n_ctas;
}
// the CTA whose range holds block b: first_block(c) <= b < first_block(c + 1)
__host__ __device__ inline int cta_of_block(long long b, long long total, int n_ctas) {
    return (int)(((b + 1) * n_ctas - 1) / total);
}

// A trace of one CTA's way through the chain (a build with -DPLM_CHAIN_TRACE only): nanoseconds since the
// kernel's start at the points marked below, [CTA][point].
#ifdef PLM_CHAIN_TRACE
__device__ unsigned long long plm_chain_trace[PLM_SM_COUNT * 2][64];
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(point) do { if (threadIdx.x == 64 && (point) < 64) plm_chain_trace[blockIdx.x][point] = trace_now(); } while (0)
__device__ unsigned long long plm_chain_blocks[4][256];      // CTA 70: per block, when W was asked for, A was asked for, the stage was full, its MMAs were issued
#define TRACE_BLOCK(kind, n) do { if (blockIdx.x == 70 && (n) < 256) plm_chain_blocks[kind][n] = trace_now(); } while (0)
#else
#define TRACE(point) do { } while (0)
#define TRACE_BLOCK(kind, n) do { } while (0)
#endif

// Whether the phase is complete, without waiting (mbarrier.try_wait may suspend the thread for a while; the
// producer has other work to look after meanwhile).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// A barrier of the four epilogue warps that also tells every one of their threads whether any of them
// brought `v`: decisions to give up are taken by all 128 threads alike, so that none is left at a barrier.
__device__ __forceinline__ bool epilogue_any(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)(v ? 1u : 0u)) : "memory");
    return r != 0;
}

// The four epilogue warps of every CTA meet: what each of their threads wrote to global memory before is
// visible to every thread of the grid after (also to TMA loads that are issued after).  Returns false if
// the wait ran out or another CTA has reported a failure.
__device__ bool meet(unsigned int* counter, unsigned int target, int* status, volatile int* s_abort) {
    epilogue_bar();                         // this CTA's writes have happened before its leader's fence
    if (threadIdx.x == 64) {
        __threadfence();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        atomicAdd(counter, 1u);
        uint32_t spins = 0;
        while (ld_acquire(counter) < target) {
            if (++spins > SPIN_LIMIT || ((spins & 63u) == 0u && *(volatile int*)status != 0)) {
                atomicCAS(status, 0, 4);
                *s_abort = 1;
                break;
            }
        }
        __threadfence();
    }
    return !epilogue_any(*s_abort != 0);
}

// A walk over one CTA's blocks of all phases in the order in which they pass through the ring.  The
// producer keeps two (weights ahead, activations behind), the MMA issuer one.  One thread steps it once per
// block, so it steps without divisions: a single thread's arithmetic is slow enough to bound the ring's rate.
struct Walk {
    int p;                      // phase (n_phases: done)
    int tile, kb, n_kb, left;   // the next block, the phase's K blocks per tile, blocks of this CTA left in the phase
    int stage;                  // the ring stage the next block goes through
    uint32_t lap;               // parity of how often the ring has been gone round
};
__device__ __forceinline__ void walk_enter(Walk& w, const Chain& ch, int cta, int n_ctas) {
    while (w.p < ch.n_phases) {                         // (skips phases in which this CTA has no block)
        const Phase& P = ch.ph[w.p];
        const long long b = first_block(P.total, cta, n_ctas), e = first_block(P.total, cta + 1, n_ctas);
        if (e > b) {
            w.n_kb = P.n_kb;
            w.tile = (int)(b / P.n_kb);
            w.kb = (int)(b - (long long)w.tile * P.n_kb);
            w.left = (int)(e - b);
            return;
        }
        ++w.p;
    }
}
template <int STAGES>
__device__ __forceinline__ void walk_step(Walk& w, const Chain& ch, int cta, int n_ctas) {
    if (++w.stage == STAGES) { w.stage = 0; w.lap ^= 1u; }
    if (--w.left == 0) {
        ++w.p;
        walk_enter(w, ch, cta, n_ctas);
    } else if (++w.kb == w.n_kb) {
        w.kb = 0;
        ++w.tile;
    }
}

#ifdef PLM_CHAIN_STAGES
template <int BN> __host__ __device__ constexpr int stages_of() { return PLM_CHAIN_STAGES; }
#else
template <int BN> __host__ __device__ constexpr int stages_of() { return BN <= 16 ? 11 : (BN <= 32 ? 10 : 8); }
#endif
template <int BN> __host__ __device__ constexpr size_t chain_smem() {
    return (size_t)stages_of<BN>() * (BM * BK * 2 + BN * BK * 2) + 1024 /*alignment*/ + 512 /*barriers*/;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
decode_chain_kernel(const __grid_constant__ Chain ch) {
    constexpr int STAGES = stages_of<BN>();
    constexpr uint32_t W_BYTES = BM * BK * 2, A_BYTES = BN * BK * 2, STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;
    const uint32_t acc_full0 = bars + 16 * STAGES, acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (acc_empty0 + 16 - raw));
    __shared__ int s_abort;
    __shared__ int s_ready;                 // phases up to this one have their input (-1: none yet)
    __shared__ float s_rstd[64];
    __shared__ float s_part[128];
    __shared__ float s_sq[MAX_SHARE];         // RESIDUAL: the squares of this CTA's share, [token][column]

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, n_ctas = gridDim.x;

    if (threadIdx.x == 0) {
        s_abort = 0;
        s_ready = -1;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);           // one arrival per epilogue warp
        }
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
        // ------------------------------------------------------------ the producer
        if (lane == 0) {
            // two walks over this CTA's blocks of all phases: the weights run ahead, the activations
            // follow as their phases' inputs come to exist
            Walk ww = {0, 0, 0, 1, 0, 0, 0u}, aw = ww;
            walk_enter(ww, ch, cta, n_ctas);
            walk_enter(aw, ch, cta, n_ctas);
            int w_n = 0, a_n = 0;                                       // blocks asked for so far
            bool waited = false;
            int fenced = -1;
            uint32_t idle = 0;
            while (ww.p < ch.n_phases || aw.p < ch.n_phases) {
                bool moved = false;
                if (ww.p < ch.n_phases && mbar_test(empty0 + 8 * ww.stage, ww.lap ^ 1u)) {
                    mbar_expect_tx(full0 + 8 * ww.stage, STAGE_BYTES);
                    tma_load_2d(base + ww.stage * STAGE_BYTES, &ch.ph[ww.p].map_w, full0 + 8 * ww.stage, ww.kb * BK, ww.tile * BM);
                    TRACE_BLOCK(0, w_n);
                    ++w_n;
                    walk_step<STAGES>(ww, ch, cta, n_ctas);
                    moved = true;
                }
                if (aw.p < ch.n_phases && a_n < w_n && *(volatile int*)&s_ready >= aw.p) {
                    if (!waited) { pdl_wait(); waited = true; }
                    if (fenced != aw.p) {   // once per phase: what other CTAs wrote before the meeting, for the copies below
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                        fenced = aw.p;
                    }
                    tma_load_2d(base + aw.stage * STAGE_BYTES + W_BYTES, &ch.ph[aw.p].map_a, full0 + 8 * aw.stage, aw.kb * BK, 0);
                    TRACE_BLOCK(1, a_n);
                    ++a_n;
                    walk_step<STAGES>(aw, ch, cta, n_ctas);
                    moved = true;
                }
                if (moved) { idle = 0; continue; }
                if (*(volatile int*)&s_abort) break;
                if (++idle > WAIT_LIMIT) { atomicCAS(ch.status, 0, 1); s_abort = 1; break; }
            }
            if (*(volatile int*)&s_abort) {
                // Weight blocks that were asked for and whose activation tile never was cannot complete
                // their stage; the copies themselves land within microseconds.  Give them that time
                // before the shared memory goes away.
                for (int i = 0; i < 2000; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- the MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            Walk cw = {0, 0, 0, 1, 0, 0, 0u};
            walk_enter(cw, ch, cta, n_ctas);
            int seg = 0, n = 0;
            bool first = true;                                          // the next block opens a segment (a tile's run of blocks)
            while (cw.p < ch.n_phases) {
                const int buf = seg & 1;
                if (*(volatile int*)&s_abort) break;
                if (first) {
                    if (!mbar_wait(acc_empty0 + 8 * buf, (uint32_t)(((seg >> 1) & 1) ^ 1), ch.status, 2)) { s_abort = 1; break; }
                    tc_fence_after();
                }
                if (!mbar_wait(full0 + 8 * cw.stage, cw.lap, ch.status, 2)) { s_abort = 1; break; }
                TRACE_BLOCK(2, n);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                const uint64_t wd = smem_desc_sw128(base + cw.stage * STAGE_BYTES);
                const uint64_t ad = smem_desc_sw128(base + cw.stage * STAGE_BYTES + W_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_bf16(d_tmem, wd + (uint64_t)(k * UMMA_K * 2 / 16), ad + (uint64_t)(k * UMMA_K * 2 / 16),
                                idesc, (!first || k > 0) ? 1u : 0u);
                tc_commit(empty0 + 8 * cw.stage);
                TRACE_BLOCK(3, n);
                ++n;
                const bool closes = cw.left == 1 || cw.kb == cw.n_kb - 1;   // the CTA's range or the tile ends here
                if (closes) {
                    tc_commit(acc_full0 + 8 * buf);
                    ++seg;
                }
                first = closes;
                walk_step<STAGES>(cw, ch, cta, n_ctas);
            }
        }
    } else {
        // ------------------------------------------- accumulators out, meetings, epilogues
        const int tid = threadIdx.x - 64;                   // 0..127
        const int quarter = warp & 3;                       // the TMEM lanes this warp may read
        const int row = quarter * 32 + lane;
        unsigned int meetings = 0;
        int seg = 0;
        bool ok = true;
        TRACE(0);
        pdl_wait();                                         // the chain's input and the stream are there
        TRACE(1);
        if (tid == 0) s_ready = 0;
        for (int p = 0; p < ch.n_phases && ok; ++p) {
            const Phase& P = ch.ph[p];
            long long b = first_block(P.total, cta, n_ctas);
            const long long e = first_block(P.total, cta + 1, n_ctas);
            while (b < e && ok) {
                const long long tile = b / P.n_kb;
                const long long seg_end = min(e, (tile + 1) * P.n_kb);
                const int buf = seg & 1;
                const bool got = mbar_wait(acc_full0 + 8 * buf, (uint32_t)((seg >> 1) & 1), ch.status, 3);
                if (!got) s_abort = 1;
                if (epilogue_any(!got || *(volatile int*)&s_abort != 0)) { ok = false; break; }
                tc_fence_after();
                const int slot = cta - cta_of_block(tile * P.n_kb, P.total, n_ctas);
                float* dst = ch.partial + (((size_t)tile * P.slots + slot) * BM + row) * BN;   // [tile][slot][row][token]
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t r[32];
                    tc_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        if (c + j < ch.T)
                            *reinterpret_cast<uint4*>(dst + c + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
                b = seg_end;
                ++seg;
            }
            if (!ok) break;
            TRACE(2 + 4 * p);
            // ---- everyone's partial sums of this phase are written
            if (!meet(ch.sync, ++meetings * (unsigned)n_ctas, ch.status, &s_abort)) { ok = false; break; }
            TRACE(3 + 4 * p);

            // ---- this CTA's share of the phase's columns: sum, epilogue, write
            const int n_cols = P.kind == KIND_SWIGLU ? P.N / 2 : P.N;
            const int c_lo = (int)((long long)n_cols * cta / n_ctas), c_hi = (int)((long long)n_cols * (cta + 1) / n_ctas);
            if (P.kind == KIND_SWIGLU || P.kind == KIND_SCALED) {
                // every token's sum of squares: the CTAs' parts are dealt over the groups of BN threads (loads of a
                // group's thread are asked for sixteen at a time), then one thread a token adds the groups' sums in order
                constexpr int GROUPS = 128 / BN;
                const int t = tid % BN, grp = tid / BN;
                float ss = 0.f;
                if (t < ch.T) {
                    for (int c0 = grp; c0 < n_ctas; c0 += 16 * GROUPS) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int c = c0 + j * GROUPS;
                            v[j] = c < n_ctas ? __ldcg(P.ss_in + (size_t)c * SS_LD + t) : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) ss += v[j];
                    }
                }
                s_part[grp * BN + t] = ss;
                epilogue_bar();
                if (tid < BN) {
                    float sum = 0.f;
#pragma unroll
                    for (int g2 = 0; g2 < GROUPS; ++g2) sum += s_part[g2 * BN + tid];
                    s_rstd[tid] = 1.0f / sqrtf(sum * P.inv_size + P.eps);
                }
                epilogue_bar();
            }
            // Four tokens of one row of a tile, summed over the tile's slots in slot order.  All loads are asked for
            // before any is added, so a thread waits for the second-level cache once, not once per slot.
            auto summed4 = [&](int tile, int r, int t4) {
                const int s0 = cta_of_block((long long)tile * P.n_kb, P.total, n_ctas);
                const int s1 = cta_of_block((long long)(tile + 1) * P.n_kb - 1, P.total, n_ctas);
                const float* src = ch.partial + (((size_t)tile * P.slots) * BM + r) * BN + t4;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sb = 0; sb <= s1 - s0; sb += 12) {
                    float4 v[12];
#pragma unroll
                    for (int j = 0; j < 12; ++j) {
                        const int s = sb + j;
                        // (with fewer blocks than CTAs, CTAs in between have no block and wrote nothing)
                        const bool there = s <= s1 - s0 &&
                            (P.total >= n_ctas || first_block(P.total, s0 + s, n_ctas) < first_block(P.total, s0 + s + 1, n_ctas));
                        v[j] = there ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)s * BM * BN))
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 12; ++j) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
                }
                return acc;
            };
            const int ncols = c_hi - c_lo, quads = (ch.T + 3) / 4, items = ncols * quads;
            for (int idx = tid; idx < items; idx += 128) {  // all (column, four tokens) pairs of the share at once
                const int qd = idx / ncols, c = c_lo + (idx - qd * ncols), t0 = qd * 4;
                float val[4], xv[4] = {0.f, 0.f, 0.f, 0.f}, nwc = 0.f;
                if (P.kind == KIND_RESIDUAL) {                  // asked for before the partial sums are waited for
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (t0 + e < ch.T) xv[e] = __ldcg(P.resid + (size_t)(t0 + e) * P.ld_resid + c);
                    nwc = __bfloat162float(P.norm_w[c]);
                }
                if (P.kind == KIND_SWIGLU) {
                    const int tile = c >> 6, r = c & 63;
                    const float4 g = summed4(tile, r, t0), u = summed4(tile, 64 + r, t0);
                    const float gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float sc = s_rstd[min(t0 + e, BN - 1)];
                        val[e] = swiglu_bf16(gs[e] * sc, us[e] * sc);
                    }
                } else {
                    const float4 v = summed4(c >> 7, c & 127, t0);
                    val[0] = v.x; val[1] = v.y; val[2] = v.z; val[3] = v.w;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = t0 + e;
                    if (t >= ch.T) break;
                    if (P.kind == KIND_RESIDUAL) {
                        const float xn = xv[e] + val[e];
                        P.resid[(size_t)t * P.ld_resid + c] = xn;
                        reinterpret_cast<bf16*>(P.out)[(size_t)t * P.ldo + c] = __float2bfloat16_rn(xn * nwc);
                        s_sq[t * ncols + (c - c_lo)] = xn * xn;
                    } else if (P.kind == KIND_PLAIN) {
                        reinterpret_cast<float*>(P.out)[(size_t)t * P.ldo + c] = val[e];
                    } else {
                        const float o = P.kind == KIND_SCALED ? val[e] * s_rstd[t] : val[e];
                        reinterpret_cast<bf16*>(P.out)[(size_t)t * P.ldo + c] = __float2bfloat16_rn(o);
                    }
                }
            }
            if (P.kind == KIND_RESIDUAL) {                  // this CTA's part of every token's sum of squares, in column order
                epilogue_bar();
                if (tid < ch.T) {
                    float sq = 0.f;
                    for (int j = 0; j < ncols; ++j) sq += s_sq[tid * ncols + j];
                    P.ss_out[(size_t)cta * SS_LD + tid] = sq;
                }
            }
            TRACE(4 + 4 * p);
            if (p + 1 < ch.n_phases) {
                // ---- the phase's output is complete everywhere: the next phase may read it
                if (!meet(ch.sync, ++meetings * (unsigned)n_ctas, ch.status, &s_abort)) { ok = false; break; }
                if (tid == 0) s_ready = p + 1;
                TRACE(5 + 4 * p);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0) {
        // the last CTA to leave puts the counters back to zero for the next launch
        __threadfence();
        if (atomicAdd(ch.sync + 1, 1u) == (unsigned)n_ctas - 1) {
            ch.sync[0] = 0u;
            ch.sync[1] = 0u;
            __threadfence();
        }
    }
}

int persistent_ctas() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = PLM_SM_COUNT;
    }
    return n;
}

template <int BN>
int launch_chain(const Chain& ch, cudaStream_t stream) {
    static bool configured = false;
    constexpr size_t smem = chain_smem<BN>();
    auto kern = decode_chain_kernel<BN>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return plm_status_of(launch_pdl(kern, dim3(persistent_ctas()), dim3(NUM_THREADS), smem, stream, ch));
}

}  // namespace

// One phase as the caller describes it.
struct PlmChainPhase {
    int kind;                   // 0 RESIDUAL, 1 SWIGLU, 2 SCALED, 3 PLAIN
    int N, K;                   // w is [N, K]
    const void* w; long long ldw;
    const void* a; long long lda;   // the phase's input [T, K] bf16 (the output of the phase before, or the chain's input)
    void* out; long long ldo;
    float* resid; long long ld_resid;
    const void* norm_w;
    float* ss_out;              // RESIDUAL: [CTAs, 64]
    const float* ss_in;         // SWIGLU, SCALED
    int size; float eps;        // the norm's width and eps
};

#ifdef PLM_CHAIN_TRACE
extern "C" int plm_chain_trace_read(unsigned long long* host, int n_ctas) {
    return plm_status_of(cudaMemcpyFromSymbol(host, plm_chain_trace, sizeof(unsigned long long) * 64 * n_ctas));
}
extern "C" int plm_chain_blocks_read(unsigned long long* host) {
    return plm_status_of(cudaMemcpyFromSymbol(host, plm_chain_blocks, sizeof(unsigned long long) * 4 * 256));
}
#endif

// How many CTAs the chain kernel runs (the rows of a sums-of-squares table).
extern "C" int plm_decode_chain_ctas() { return persistent_ctas(); }

// Floats of partial-sum scratch that a phase of (N, K) needs for up to `T` tokens.
extern "C" long long plm_decode_chain_scratch(int N, int K, int T) {
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    const int n_ctas = persistent_ctas();
    const long long n_tiles = (N + BM - 1) / BM, n_kb = (K + BK - 1) / BK, total = n_tiles * n_kb;
    int slots = 1;
    for (long long t = 0; t < n_tiles; ++t) {
        const int s = cta_of_block((t + 1) * n_kb - 1, total, n_ctas) - cta_of_block(t * n_kb, total, n_ctas) + 1;
        if (s > slots) slots = s;
    }
    return n_tiles * slots * bn * BM;
}

// Run `n` phases (2..4) for T <= 64 tokens.  `partial`: scratch of at least the largest phase's
// plm_decode_chain_scratch floats; `sync`: two unsigned ints that are zero (the kernel leaves them zero).
extern "C" int plm_decode_chain(const PlmChainPhase* phases, int n, int T, float* partial, unsigned int* sync,
                                int* status, cudaStream_t stream) {
    if (n < 1 || n > MAX_PHASES || T <= 0 || T > 64) return PLM_ERR_SHAPE;
    if (!partial || !sync || !status) return PLM_ERR_SHAPE;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    const int n_ctas = persistent_ctas();
    Chain ch = {};
    ch.n_phases = n;
    ch.T = T;
    ch.partial = partial;
    ch.sync = sync;
    ch.status = status;
    for (int i = 0; i < n; ++i) {
        const PlmChainPhase& in = phases[i];
        Phase& P = ch.ph[i];
        if (in.kind < 0 || in.kind > 3 || in.N <= 0 || in.K <= 0 || !in.w || !in.a || !in.out) return PLM_ERR_SHAPE;
        if (in.K % 8 || in.ldw % 8 || in.lda % 8 || (((uintptr_t)in.w | (uintptr_t)in.a) & 15)) return PLM_ERR_ALIGN;
        if (in.kind == KIND_SWIGLU && in.N % 128) return PLM_ERR_SHAPE;
        if (in.kind == KIND_RESIDUAL && (!in.resid || !in.norm_w || !in.ss_out)) return PLM_ERR_SHAPE;
        if (in.kind == KIND_RESIDUAL && (long long)T * ((in.N + n_ctas - 1) / n_ctas + 1) > MAX_SHARE) return PLM_ERR_UNSUPPORTED;
        if ((in.kind == KIND_SWIGLU || in.kind == KIND_SCALED) && (!in.ss_in || in.size <= 0)) return PLM_ERR_SHAPE;
        int rc;
        if ((rc = make_map(&P.map_w, in.w, in.N, in.K, in.ldw, BM)) != PLM_OK) return rc;
        if ((rc = make_map(&P.map_a, in.a, T, in.K, in.lda, bn)) != PLM_OK) return rc;
        P.kind = in.kind; P.N = in.N; P.K = in.K;
        P.n_tiles = (in.N + BM - 1) / BM;
        P.n_kb = (in.K + BK - 1) / BK;
        P.total = (long long)P.n_tiles * P.n_kb;
        int slots = 1;
        for (long long t = 0; t < P.n_tiles; ++t) {
            const int s = cta_of_block((t + 1) * P.n_kb - 1, P.total, n_ctas) - cta_of_block(t * P.n_kb, P.total, n_ctas) + 1;
            if (s > slots) slots = s;
        }
        P.slots = slots;
        P.out = in.out; P.ldo = in.ldo;
        P.resid = in.resid; P.ld_resid = in.ld_resid;
        P.norm_w = (const bf16*)in.norm_w;
        P.ss_out = in.ss_out; P.ss_in = in.ss_in;
        P.inv_size = in.size > 0 ? 1.0f / (float)in.size : 0.f;
        P.eps = in.eps;
    }
    if (bn == 16) return launch_chain<16>(ch, stream);
    if (bn == 32) return launch_chain<32>(ch, stream);
    return launch_chain<64>(ch, stream);
}
