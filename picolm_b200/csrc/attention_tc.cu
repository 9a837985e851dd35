// Causal prefill attention over the paged cache on the fifth-generation tensor
// cores, compiled for one head size (-DPLM_HD = 64 or 128).
//
// One CTA takes 128 query tokens of one head and walks that sequence's pages of
// 64 keys.  Per page:
//   S = Q K^T      tcgen05.mma, Q and K in shared memory (TMA, 128-byte swizzle), S in TMEM
//   softmax        one thread per query row: tcgen05.ld its 64 scores, scale, mask, running
//                  max / sum in fp32 (the recurrence of picolm/model_attention.c:43-140 taken a
//                  page at a time), probabilities back to TMEM as bf16 (tcgen05.st)
//   O += P V       tcgen05.mma with P from TMEM and V in shared memory (MN-major), accumulating in
//                  TMEM across pages; O is rescaled only when a row's maximum has outgrown the
//                  reference it is kept against by a factor of 256
// Warp 0 loads (TMA), warp 1 issues the MMAs and owns the tensor memory, warps 2..5 are the
// 128 softmax threads.  The scores have two buffers in TMEM.  As soon as all 128 threads have handed
// over P(i), and with that have read S(i), the issuing thread puts Q K(i + 2)^T into the freed buffer
// and only then P(i) V(i), so the scores of the pages ahead are there when the softmax threads get to
// them.  (With head size 128 the output takes half of the CTA's tensor memory; P(i) is then written over
// S(i) and P(i) V(i) goes first.)  The softmax warps may drift up to a page apart (never two: page i + 2
// needs what follows everybody's arrival for page i), so even and odd pages count their arrivals on
// barriers of their own.  Keys of a KV head are shared by its
// query heads through L2 (consecutive CTAs work on the heads of one group).
//
// Waits on mbarriers are bounded as in gemm_tc.cu: a wait that runs out records where in
// `status`, the CTA stops issuing work, lets what is in flight land, frees its TMEM and returns.
#include "tc_common.cuh"

#ifndef PLM_HD
#define PLM_HD 64
#endif

using namespace plm_tc;

namespace {

constexpr int HD = PLM_HD;
static_assert(HD == 64 || HD == 128, "the tcgen05 attention is built for head sizes 64 and 128");
constexpr int CB = HD / 64;                       // 64-column blocks of a row (one 128-byte swizzle span each)
constexpr int BQ = 128, BKV = 64;
constexpr int KS = HD == 64 ? 4 : 2, VS = KS;    // tiles of keys and of values in shared memory
// With head size 128 there is room for two tiles of each, and the scores are issued two pages ahead: keys and
// values then have rings of their own (a key tile is free after Q K^T, a value tile only after P V, two pages
// later).  With head size 64 a page's keys and values arrive on one barrier and are given back together: the
// second ring's waits and commits cost the issuing thread more than four tiles of each leave to gain.
constexpr bool SPLIT_RINGS = HD == 128;
constexpr int NSB = 2;                            // score buffers in TMEM
// With head size 128 the output takes half of the CTA's tensor memory (two CTAs an SM, 256 columns each), so
// the probabilities of a page are written over its own scores: a thread has read its row of S before it
// writes its row of P, and P takes the first 32 of the buffer's 64 columns.
constexpr bool P_OVER_S = HD == 128;
constexpr uint32_t Q_BLOCK = BQ * 128, KV_BLOCK = BKV * 128;       // bytes of one 64-column block
constexpr uint32_t Q_BYTES = CB * Q_BLOCK, K_BYTES = CB * KV_BLOCK, V_BYTES = K_BYTES;
constexpr uint32_t TM_S = 0, TM_P = NSB * 64, TM_PV = P_OVER_S ? TM_P : TM_P + 2 * 32, TMEM_COLS = 256;
static_assert(TM_PV + HD <= TMEM_COLS, "TMEM budget");
static_assert(SPLIT_RINGS ? (KS >= NSB && VS >= 2) : KS > NSB,
              "the scores of page i + NSB are issued while page i still holds its values");
constexpr size_t SMEM = Q_BYTES + KS * K_BYTES + VS * V_BYTES + 1024 + 256;
constexpr float LOG2E = 1.4426950408889634f;

// Latency-critical waits (a handoff per page between the MMA issuer and the softmax threads): poll
// with test_wait, which returns at once, instead of try_wait, which may park the thread for a while.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, int* status, int where) {
    for (uint32_t i = 0; i < (1u << 26); ++i)
        if (mbar_test(bar, parity)) return true;
    if (status) atomicCAS(status, 0, where);
    return false;
}
// 2^x by the special-function unit; 2^(-inf) = 0
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two fp32 lanes per instruction (fma.rn.f32x2 and add.rn.f32x2 round each lane as the scalar forms do) and
// the three-input maximum: the softmax threads are bound by how many instructions a key costs them.
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// V tile [64 keys][64 columns] per block, 128-byte rows with TMA's 128-byte swizzle, used as the B
// operand with N (the head's columns) contiguous: MN-major.  8-key groups are 1024 bytes apart
// (stride offset), 64-column blocks KV_BLOCK bytes apart (leading offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(KV_BLOCK >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D fp32, A and B bf16, M = 128, N = n; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BQ >> 4) << 24);
}

// A build with -DPLM_ATTN_TRACE records the SM's cycle counter at the points marked ATTN_TRACE below, for the
// first 128 pages of the CTA that starts first: rows 0..3 of the table for the four softmax warps (0 scores
// seen, 1 scores in registers, 2 maximum known and P's place free, 3 exponentials done, 4 P in tensor memory,
// 5 arrived), row 4 for the issuing thread (0 everybody's arrival seen, 1 first group of MMAs issued, 2 both
// issued and committed).  plm_attn_tc_trace_read copies the table out.  A point costs the thread that passes
// it some tens of cycles, so the traced CTA runs a little slower than the others.
#ifdef PLM_ATTN_TRACE
constexpr int TRACE_PAGES = 128;
__device__ long long plm_attn_trace[5][TRACE_PAGES][8];
#define ATTN_TRACE(who, page, point)                                                                      \
    do { if (traced && (page) < TRACE_PAGES) plm_attn_trace[who][page][point] = clock64(); } while (0)
#else
#define ATTN_TRACE(who, page, point) do { } while (0)
#endif

// grid = (query tiles of the longest sequence, heads, sequences)
__global__ void __launch_bounds__(NUM_THREADS, 2)
attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_kv_len,
                       const int* __restrict__ block_table, int max_pages, int H, int G, float scale_log2, int window,
                       int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t q_smem = base, k_smem0 = base + Q_BYTES, v_smem0 = k_smem0 + KS * K_BYTES;
    const uint32_t bars = v_smem0 + VS * V_BYTES;
    const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = k_full0 + 8 * KS,
                   v_full0 = SPLIT_RINGS ? k_empty0 + 8 * KS : k_full0, v_empty0 = SPLIT_RINGS ? v_full0 + 8 * VS : k_empty0,
                   s_full0 = k_empty0 + 8 * KS + 16 * VS, p_ready0 = s_full0 + 8 * NSB,
                   pv_full0 = p_ready0 + 16;                              // p_ready[2], pv_full[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (pv_full0 + 16 - raw));
    __shared__ int s_abort;

    pdl_launch_dependents();
    // Blocks start in the order of their index (x fastest): the longest query tiles (those at the end of
    // a sequence, which see the most keys) of all heads first, the short ones fill the end.  Heads of
    // one KV head are neighbours, so they stream the same keys at about the same time.
    const int b = blockIdx.z;
    const int lin = blockIdx.y * gridDim.x + blockIdx.x;
    const int h = lin % H, rank_of_tile = lin / H;
    const int t0 = seq_start[b], n_new = seq_start[b + 1] - t0;          // inputs written before the step began
    const int n_tiles = (n_new + BQ - 1) / BQ;
    if (rank_of_tile >= n_tiles) return;
    const int tile = n_tiles - 1 - rank_of_tile;
    const int kv_len = PLM_POSITION(seq_kv_len[b] - 1) + 1;
    const int pos0 = kv_len - n_new + tile * BQ;                         // position of the tile's first row
    const int rows = min(BQ, n_new - tile * BQ);
    const int g = h / (H / G);
    const int pos_last = pos0 + rows - 1;
    const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int page_first = first_key / BKV, page_last = pos_last / BKV;
    const int n_pages = page_last - page_first + 1;
    const int* pages = block_table + (size_t)b * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef PLM_ATTN_TRACE
    const bool traced = lin == 0 && b == 0 && lane == 0 && warp >= 1;
    const int softmax_warp = warp - 2;
#endif

    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < KS; ++s) { mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1); }
        if (SPLIT_RINGS)
            for (int s = 0; s < VS; ++s) { mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1); }
        for (int s = 0; s < NSB; ++s) mbar_init(s_full0 + 8 * s, 1);
        mbar_init(p_ready0, 128);
        mbar_init(p_ready0 + 8, 128);
        mbar_init(pv_full0, 1);
        mbar_init(pv_full0 + 8, 1);
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
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            pdl_wait();                                                  // q and the new keys come from the kernel before
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int cb = 0; cb < CB; ++cb)
                tma_load_2d(q_smem + cb * Q_BLOCK, &map_q, q_full, h * HD + cb * 64, t0 + tile * BQ);
            int issued_k = 0, issued_v = 0;
            for (int i = 0; i < n_pages; ++i) {
                const int ks = i % KS, vs = i % VS;
                const int row = (PLM_PAGE_NO(pages[page_first + i]) * G + g) * BKV;
                if (*(volatile int*)&s_abort) break;
                if (!mbar_wait(k_empty0 + 8 * ks, ((i / KS) & 1) ^ 1, status, 1)) { s_abort = 1; break; }
                mbar_expect_tx(k_full0 + 8 * ks, SPLIT_RINGS ? K_BYTES : K_BYTES + V_BYTES);
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    tma_load_2d(k_smem0 + ks * K_BYTES + cb * KV_BLOCK, &map_k, k_full0 + 8 * ks, cb * 64, row);
                issued_k = i + 1;
                if (SPLIT_RINGS) {
                    if (!mbar_wait(v_empty0 + 8 * vs, ((i / VS) & 1) ^ 1, status, 1)) { s_abort = 1; break; }
                    mbar_expect_tx(v_full0 + 8 * vs, V_BYTES);
                }
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    tma_load_2d(v_smem0 + vs * V_BYTES + cb * KV_BLOCK, &map_v, v_full0 + 8 * vs, cb * 64, row);
                issued_v = i + 1;
            }
            if (*(volatile int*)&s_abort) {                              // let what is in flight land
                mbar_wait(q_full, 0, nullptr, 0);
                for (int i = max(0, issued_k - KS); i < issued_k; ++i)
                    mbar_wait(k_full0 + 8 * (i % KS), (i / KS) & 1, nullptr, 0);
                if (SPLIT_RINGS)
                    for (int i = max(0, issued_v - VS); i < issued_v; ++i)
                        mbar_wait(v_full0 + 8 * (i % VS), (i / VS) & 1, nullptr, 0);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(BKV, false), idesc_o = instr_desc(HD, true);
            auto qk = [&](int i) {                                       // S[i % NSB] = Q K(i)^T
                const uint32_t k_smem = k_smem0 + (i % KS) * K_BYTES;
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_bf16(tmem + TM_S + (i % NSB) * 64,
                                    smem_desc_sw128(q_smem + cb * Q_BLOCK) + (uint64_t)(k * 2),
                                    smem_desc_sw128(k_smem + cb * KV_BLOCK) + (uint64_t)(k * 2), idesc_s,
                                    (cb > 0 || k > 0) ? 1u : 0u);
                tc_commit(s_full0 + 8 * (i % NSB));
                if (SPLIT_RINGS) tc_commit(k_empty0 + 8 * (i % KS));
            };
            bool ok = mbar_wait(q_full, 0, status, 2);
            for (int j = 0; j < NSB && j < n_pages && ok; ++j) {         // fill the score buffers
                ok = mbar_wait(k_full0 + 8 * (j % KS), (j / KS) & 1, status, 2);
                if (ok) { tc_fence_after(); qk(j); }
            }
            for (int i = 0; i < n_pages && ok; ++i) {
                if (*(volatile int*)&s_abort) { ok = false; break; }
                if (!mbar_spin(p_ready0 + 8 * (i & 1), (i >> 1) & 1, status, 2)) { ok = false; break; }
                tc_fence_after();
                ATTN_TRACE(4, i, 0);
                // The softmax threads have read S(i): its buffer takes the scores of page i + NSB at once, before
                // P(i) V(i) is issued, so that they are there when the softmax of the page in between is done.
                // Where P(i) lies in that buffer, P(i) V(i) goes first: the MMAs of one thread run in their order.
                auto scores_ahead = [&]() {
                    const int nxt = i + NSB;
                    if (nxt >= n_pages) return true;
                    if (!mbar_wait(k_full0 + 8 * (nxt % KS), (nxt / KS) & 1, status, 2)) return false;
                    tc_fence_after();
                    qk(nxt);
                    return true;
                };
                if (!P_OVER_S && !scores_ahead()) { ok = false; break; }
                if (!P_OVER_S) ATTN_TRACE(4, i, 1);
                if (SPLIT_RINGS) {
                    if (!mbar_wait(v_full0 + 8 * (i % VS), (i / VS) & 1, status, 2)) { ok = false; break; }
                    tc_fence_after();
                }
                const uint32_t v_smem = v_smem0 + (i % VS) * V_BYTES;
                const uint32_t p_tmem = P_OVER_S ? TM_S + (i % NSB) * 64 : TM_P + (i & 1) * 32;
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)                       // O_page = P V(i), 16 keys a step
                    tc_mma_bf16_ts(tmem + TM_PV, tmem + p_tmem + k * 8, smem_desc_sw128_mn(v_smem + k * 2048), idesc_o,
                                   (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(pv_full0 + 8 * (i & 1));                     // P buffer i % 2 is free, O holds pages 0..i
                tc_commit(v_empty0 + 8 * (i % VS));
                if (P_OVER_S) ATTN_TRACE(4, i, 1);
                if (P_OVER_S && !scores_ahead()) { ok = false; break; }
                ATTN_TRACE(4, i, 2);
            }
            if (!ok) s_abort = 1;
        }
    } else {
        // ----------------------------------------------------------------- softmax
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                               // this thread's query row
        const int pos = r < rows ? pos0 + r : -1;                        // -1: no such row, everything masked
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        // O stays in tensor memory and the MMAs accumulate into it across pages.  Probabilities are
        // taken relative to a reference maximum m_ref that is raised (and O rescaled) only when a
        // row's maximum outgrows it by more than 2^RESCALE_LOG2, so most pages need no pass over O.
        constexpr float RESCALE_LOG2 = 8.f;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_pages && ok; ++i) {
            if (!mbar_spin(s_full0 + 8 * (i % NSB), (i / NSB) & 1, status, 3)) { ok = false; break; }
            tc_fence_after();
            ATTN_TRACE(softmax_warp, i, 0);
            const int key0 = (page_first + i) * BKV;
            const bool need_mask = key0 + BKV - 1 > pos0 || key0 < (window > 0 ? pos_last - window + 1 : 0);
            float mx = -INFINITY;
            uint32_t s0[32], s1[32];
            tc_ld32(tmem + lane_bits + TM_S + (i % NSB) * 64, s0);
            tc_ld32(tmem + lane_bits + TM_S + (i % NSB) * 64 + 32, s1);
            tc_wait_ld();
            ATTN_TRACE(softmax_warp, i, 1);
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int ka = key0 + j, kc2 = key0 + 32 + j;
                    if (ka > pos || ka < lo) s0[j] = 0xff800000u;        // -inf
                    if (kc2 > pos || kc2 < lo) s1[j] = 0xff800000u;
                }
            } else if (pos < 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) { s0[j] = 0xff800000u; s1[j] = 0xff800000u; }
            }
            float mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;           // four chains instead of one of 32 links
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                mx = max3(mx, __uint_as_float(s0[j]), __uint_as_float(s1[j]));
                mx1 = max3(mx1, __uint_as_float(s0[j + 1]), __uint_as_float(s1[j + 1]));
                mx2 = max3(mx2, __uint_as_float(s0[j + 2]), __uint_as_float(s1[j + 2]));
                mx3 = max3(mx3, __uint_as_float(s0[j + 3]), __uint_as_float(s1[j + 3]));
            }
            mx = fmaxf(fmaxf(mx, mx1), fmaxf(mx2, mx3));
            // the scale is positive, so the maximum of the scaled scores is the scaled maximum
            const float m_cand = fmaxf(m_ref, mx * scale_log2);
            const bool raise = m_cand > m_ref + RESCALE_LOG2 || (m_ref == -INFINITY && m_cand > -INFINITY);
            // P has two buffers: page i writes the one that page i - 2 used, whose P V must be done.  (Written over
            // the scores it is: S(i) was issued after P(i - 2) V(i - 2) by the same thread.)
            if (!P_OVER_S && i > 1 && !mbar_spin(pv_full0 + 8 * (i & 1), ((i - 2) >> 1) & 1, status, 3)) { ok = false; break; }
            if (__any_sync(0xffffffffu, raise)) {                        // tcgen05.ld/st are warp-wide
                const float alpha = raise ? ex2(m_ref - m_cand) : 1.f;   // m_ref = -inf gives 0
                if (i > 0) {
                    // O may only be touched once every P V issued so far has landed in it
                    if (!mbar_spin(pv_full0 + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, status, 3)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t ov[32];
                        tc_ld32(tmem + lane_bits + TM_PV + c, ov);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
                        tc_st32(tmem + lane_bits + TM_PV + c, ov);
                    }
                }
                if (raise) { l *= alpha; m_ref = m_cand; }
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            ATTN_TRACE(softmax_warp, i, 2);
            uint32_t p[32];
            const uint64_t scale2 = pack2(__float_as_uint(scale_log2), __float_as_uint(scale_log2));
            const uint64_t neg_m2 = pack2(__float_as_uint(-m_use), __float_as_uint(-m_use));
            uint64_t sum2 = 0;                                           // two partial sums, (0.f, 0.f)
#pragma unroll
            for (int j = 0; j < 16; ++j) {                              // p = 2^(s * scale - m_ref): half an FFMA2 and one EX2 each
                float xa0, xa1, xc0, xc1;
                unpack2(fma2(pack2(s0[2 * j], s0[2 * j + 1]), scale2, neg_m2), xa0, xa1);
                unpack2(fma2(pack2(s1[2 * j], s1[2 * j + 1]), scale2, neg_m2), xc0, xc1);
                const float a0 = ex2(xa0), a1 = ex2(xa1), c0 = ex2(xc0), c1 = ex2(xc1);
                sum2 = add2(sum2, add2(pack2(__float_as_uint(a0), __float_as_uint(a1)),
                                       pack2(__float_as_uint(c0), __float_as_uint(c1))));
                __nv_bfloat162 pa = __floats2bfloat162_rn(a0, a1), pc = __floats2bfloat162_rn(c0, c1);
                p[j] = *reinterpret_cast<uint32_t*>(&pa);               // keys 2j, 2j+1
                p[16 + j] = *reinterpret_cast<uint32_t*>(&pc);          // keys 32+2j, 32+2j+1
            }
            float sum_lo, sum_hi;
            unpack2(sum2, sum_lo, sum_hi);
            const float sum = sum_lo + sum_hi;
            l += sum;
            ATTN_TRACE(softmax_warp, i, 3);
            tc_st32(tmem + lane_bits + (P_OVER_S ? TM_S + (i % NSB) * 64 : TM_P + (i & 1) * 32), p);
            tc_wait_st();
            ATTN_TRACE(softmax_warp, i, 4);
            // places of the sequence's last page that hold no key yet: zero those rows of V, so that
            // whatever an earlier owner of the page left there cannot reach the sum (0 * NaN)
            const int valid = kv_len - key0;
            if (valid < BKV) {
                ok = mbar_wait(v_full0 + 8 * (i % VS), (i / VS) & 1, status, 3);
                uint8_t* v_ptr = smem_raw + (v_smem0 + (i % VS) * V_BYTES - raw);
                for (int idx = (int)threadIdx.x - 64; idx < (BKV - valid) * CB * 8; idx += 128) {
                    const int row = valid + idx / (CB * 8), rest = idx % (CB * 8);
                    *reinterpret_cast<uint4*>(v_ptr + (rest / 8) * KV_BLOCK + row * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tc_fence_before();
            // Even and odd pages count their arrivals on barriers of their own: a warp may be a page ahead of
            // another (never two: page i + 2 needs P V(i), which needs everybody's arrival for page i), and its
            // arrival must not be counted among those of the page before.
            mbar_arrive(p_ready0 + 8 * (i & 1));
            ATTN_TRACE(softmax_warp, i, 5);
        }
        if (ok && !mbar_spin(pv_full0 + 8 * ((n_pages - 1) & 1), ((n_pages - 1) >> 1) & 1, status, 3)) ok = false;
        tc_fence_after();
        if (!ok) s_abort = 1;
        if (ok) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + ((size_t)(t0 + tile * BQ + r) * H + h) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t ov[32];
                tc_ld32(tmem + lane_bits + TM_PV + c, ov);                // warp-wide, also for rows that are not written
                tc_wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(ov[d + 2 * j]) * inv,
                                                                      __uint_as_float(ov[d + 2 * j + 1]) * inv);
                            w[j] = *reinterpret_cast<uint32_t*>(&v2);
                        }
                        *reinterpret_cast<uint4*>(dst + c + d) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

extern "C" int plm_attn_tc_head_dim() { return HD; }

#ifdef PLM_ATTN_TRACE
// [5][128][8] cycle counts of the last launch's first CTA (see ATTN_TRACE above)
extern "C" int plm_attn_tc_trace_read(void* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, plm_attn_trace, sizeof(plm_attn_trace));
}
#endif

// q [T, H, HD] bf16, k/v cache [n_pages, G, 64, HD] bf16, out [T, H*HD] bf16.  seq_start [B+1]:
// offsets of each sequence's new tokens; seq_kv_len [B]: its length after the step; max_new: the most
// new tokens of a sequence.  `status`: a device int that stays 0 unless a bounded wait ran out.
extern "C" int plm_attn_tc_prefill(const void* q, const void* kc, const void* vc, void* out, const int* seq_start,
                                   const int* seq_kv_len, const int* block_table, int max_pages, int n_pages,
                                   int n_tokens, int n_seqs, int max_new, int H, int G, float scale, int window,
                                   int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0 || n_tokens <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || H % G || n_seqs > 65535 || H > 65535) return PLM_ERR_SHAPE;
    if ((((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out)) & 15) return PLM_ERR_ALIGN;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_map(&mq, q, n_tokens, (long)H * HD, (long)H * HD, BQ)) != PLM_OK) return rc;
    if ((rc = make_map(&mk, kc, (long)n_pages * G * BKV, HD, HD, BKV)) != PLM_OK) return rc;
    if ((rc = make_map(&mv, vc, (long)n_pages * G * BKV, HD, HD, BKV)) != PLM_OK) return rc;
    dim3 grid((max_new + BQ - 1) / BQ, H, n_seqs);
    return plm_status_of(launch_pdl(attn_tc_prefill_kernel, grid, dim3(NUM_THREADS), SMEM, stream, mq, mk, mv, (bf16*)out,
                                    seq_start, seq_kv_len, block_table, max_pages, H, G, scale * LOG2E, window, status));
}
