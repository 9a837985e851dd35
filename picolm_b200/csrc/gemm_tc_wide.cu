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
//               picolm/model_core.c:3120 and 3201)
// Warp 0 loads (TMA), warp 1 issues the MMAs and owns the tensor memory, warps 2..5 are the
// epilogue.  Waits on mbarriers are bounded; a wait that runs out records where in `status`
// and the CTA drains and leaves.
//
// The epilogue.  A thread holds one token's row of the accumulator, 32 columns at a time (the next 32 are
// on their way out of tensor memory meanwhile).  Where the result's rows are 16-byte aligned it writes them
// into a piece of 128 rows x 128 bytes in shared memory, laid out as the copy engine wants it (128-byte
// swizzle), and one thread hands the piece over: a tensor store, or for EPI_RESIDUAL a tensor reduce-add, so
// that the add happens where the stream lives and its old values never come to the SM.  Otherwise each warp
// turns its 32 rows over in shared memory so that a quarter of a warp writes (or reads, adds to and writes)
// 128 consecutive bytes of one row.
//
// K splits (single CTAs, store epilogue): where a problem has fewer tiles than SMs (prompts of a few
// hundred tokens), every tile's K range is cut into `k_splits` parts that are units of work of their own;
// each writes its fp32 partial tile to its own slice of a scratch buffer, and a second kernel adds the
// slices up in order and converts.
//
// PAIR: two CTAs of a cluster (two SMs) work on one tile of 256 tokens x 256 features with
// tcgen05.mma.cta_group::2.  Each CTA loads its 128 token rows and HALF of the weight tile (128
// features), the tensor cores of both SMs read both halves, and each CTA's tensor memory receives
// its own 128 rows of the result.  What bounds these kernels is the NUMBER of tensor copies: a copy keeps
// the SM's copy engine busy for about 190 cycles plus 6.6 a KB, and two copies of 16 KB per 64 columns of K
// took longer than those columns' MMAs (512 cycles).  A pair's stage therefore holds two 64-column tiles of K
// per operand, each operand's brought in by one copy (a 3-D tensor map, see make_map).  The
// CTA of rank 0 issues all MMAs: both CTAs' loads signal ITS "full" barriers (expect-tx set there),
// its commits arrive at the "empty" and "accumulator full" barriers of both CTAs (commit with
// multicast), and both CTAs' epilogues arrive at ITS "accumulator empty" barriers.  No TMA load
// uses multicast.
#include <cstring>

#include "tc_common.cuh"

using namespace plm_tc;

namespace {

constexpr int EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2;
constexpr int TURN_LD = 36;                                  // floats per row of a warp's 32 x 32 piece: 16-byte rows, no bank conflicts
constexpr size_t TURN_BYTES = 4 * 32 * TURN_LD * 4;          // for the four epilogue warps

__host__ __device__ constexpr int stages_of(int bn) { return bn >= 256 ? 4 : 6; }
// The add to the stream leaves the tile to the copy engine, 128 rows x 32 columns of floats at a time (16 KB, two
// of them in turn); the other epilogues turn their pieces over in TURN_BYTES.  Both start where the ring ends.
constexpr size_t OUT_PIECE = (size_t)BM * 32 * 4, OUT_BYTES = 2 * OUT_PIECE;
__host__ __device__ constexpr size_t epilogue_smem(int) { return OUT_BYTES > TURN_BYTES ? OUT_BYTES : TURN_BYTES; }
__host__ __device__ constexpr size_t wide_smem(int bn, int epi) {
    return (size_t)stages_of(bn) * (BM * BK * 2 + bn * BK * 2) + 1024 + 256 + epilogue_smem(epi);
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// --- the forms for a pair of CTAs (cta_group::2); `bar` of the first three is a shared::cluster address
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// rows from `row`, all 64 columns, slabs of K from `slab` (a map of make_map with slabs > 1)
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row, int slab) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(0), "r"(row), "r"(slab) : "memory");
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
constexpr int PAIR_SLABS = 2;                                // tiles of 64 columns of K per stage and copy
__host__ __device__ constexpr int pair_stages() { return 3; }
__host__ __device__ constexpr size_t pair_smem(int epi) {
    return (size_t)pair_stages() * PAIR_SLABS * (BM * BK * 2 + 128 * BK * 2) + 1024 + 256 + epilogue_smem(epi);
}

// ---------------------------------------------------------------- the work of a CTA
// A CTA walks over pieces of work, each a range of K blocks of one output tile.  Two ways to hand them out:
//   units   (tile, part of K) number first, first + step, ...; every part of K is a piece of its own whose
//           result goes to its slice of the output (k_splits == 1: whole tiles)
//   stream  all K blocks of all tiles in a row, cut into one equal range per CTA.  A range starts and ends
//           anywhere, so all SMs work to the end whatever the number of tiles.  The CTA whose range holds a
//           tile's first K block owns the tile; a CTA that starts inside a tile leaves its part (fp32) in its
//           own slot of a workspace and raises its flag; the owner adds the parts of the CTAs after it, in
//           their order, and writes the tile.  A part is the FIRST piece of its CTA and an owner's tile its
//           LAST, and a part waits for nothing: no cycle of waits.
constexpr int PIECE_WHOLE = 0, PIECE_PART = 1, PIECE_OWNER = 2;
// The stream walk's code is in a build of its own (-DPLM_WIDE_STREAM, the library variant "gemm_tc_wide@stream"):
// with it in, the epilogue of every kernel here was 2 .. 3 us slower (registers), and most shapes never walk.
#ifdef PLM_WIDE_STREAM
constexpr bool STREAM_BUILD = true;
#else
constexpr bool STREAM_BUILD = false;
#endif

// A build with -DPLM_WIDE_TRACE records when (globaltimer, ns) each CTA of the single-CTA form passed the points
// marked WIDE_TRACE below; plm_gemm_tc_wide_trace_read copies the table out.
#ifdef PLM_WIDE_TRACE
__device__ unsigned long long plm_wide_trace[PLM_SM_COUNT][16];
#define WIDE_TRACE(point)                                                                              \
    do {                                                                                               \
        unsigned long long t_;                                                                         \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                         \
        if (blockIdx.x < PLM_SM_COUNT && (point) < 16) plm_wide_trace[blockIdx.x][point] = t_; \
    } while (0)
#define WIDE_TRACE_VALUE(point, v) do { if (blockIdx.x < PLM_SM_COUNT) plm_wide_trace[blockIdx.x][point] = (v); } while (0)
#define WIDE_TRACE_CLOCK(var) long long var = clock64()
#else
#define WIDE_TRACE(point) do { } while (0)
#define WIDE_TRACE_VALUE(point, v) do { } while (0)
#define WIDE_TRACE_CLOCK(var) do { } while (0)
#endif
struct Piece { int tile, ks, kb_begin, kb_end, kind; long tile_end; };
struct Walk {
    bool stream;
    int n_kb, n_tiles_mn, kb_per_split;
    int unit, unit_end, unit_step;                                       // units
    long pos, hi;                                                        // stream
    __host__ __device__ bool next(Piece& w) {
        if (stream) {
            if (pos >= hi) return false;
            w.tile = (int)(pos / n_kb);
            w.ks = 0;
            w.kb_begin = (int)(pos - (long)w.tile * n_kb);
            w.tile_end = (long)(w.tile + 1) * n_kb;
            const long e = hi < w.tile_end ? hi : w.tile_end;
            w.kb_end = w.kb_begin + (int)(e - pos);
            w.kind = w.kb_begin > 0 ? PIECE_PART : (e < w.tile_end ? PIECE_OWNER : PIECE_WHOLE);
            pos = e;
            return true;
        }
        if (unit >= unit_end) return false;
        w.tile = unit % n_tiles_mn;
        w.ks = unit / n_tiles_mn;
        w.kb_begin = w.ks * kb_per_split;
        w.kb_end = n_kb < w.kb_begin + kb_per_split ? n_kb : w.kb_begin + kb_per_split;
        w.kind = PIECE_WHOLE;
        unit += unit_step;
        return true;
    }
};
// where CTA `cta` of `ctas` starts in the row of `total` K blocks
__host__ __device__ inline long stream_begin(long total, int ctas, int cta) { return total * cta / ctas; }

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the four epilogue warps

// out[rows from `row`, columns from `col`] += the 128 x 32 floats at `src` (rows of 128 bytes, 128-byte swizzle), by the
// copy engine: the add happens where the data lives, and nothing of `out` comes to this SM.  Rows and columns beyond
// the tensor's edges are left out.  One thread; the copies of a thread form groups that it can wait for.
__device__ __forceinline__ void copy_add_out(const CUtensorMap* map, uint32_t src, int col, int row) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)map), "r"(src), "r"(col), "r"(row) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// the same as a plain store (16-bit types: 128 x 64 elements)
__device__ __forceinline__ void copy_store_out(const CUtensorMap* map, uint32_t src, int col, int row) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)map), "r"(src), "r"(col), "r"(row) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// 32 floats as 32 bf16 (64 bytes) into chunks chunk0 .. chunk0 + 3 of row `row` of a piece with 128-byte swizzle
__device__ __forceinline__ void stage_bf16(uint8_t* piece, int row, int chunk0, const uint32_t* r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * k]), __uint_as_float(r[8 * i + 2 * k + 1]));
            w[k] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(piece + row * 128 + (((chunk0 + i) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}
// wait until all but the `N` latest groups of this thread's copies have read their shared memory
template <int N> __device__ __forceinline__ void copies_have_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void copies_done() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_for_copies() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// A part in the workspace: [column / 4][row 0..127][4], so that the 32 rows of a warp lie side by side.
__device__ __forceinline__ size_t part_offset(int row, int col) { return ((size_t)(col >> 2) * BM + row) * 4; }

// --- a warp's 32 rows x 32 (fp32) or 64 (bf16) columns, turned over in shared memory: a thread holds a row,
// --- but a quarter of a warp writes 128 consecutive bytes of one row
__device__ __forceinline__ void turn_put_f32(float* turn, int lane, const uint32_t* r) {
#pragma unroll
    for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<uint4*>(turn + lane * TURN_LD + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
}
// 32 floats as bf16 into the first or second half of the thread's row
__device__ __forceinline__ void turn_put_bf16(float* turn, int lane, int half, const uint32_t* r) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
#pragma unroll
    for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<uint4*>(turn + lane * TURN_LD + half * 16 + i) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
}
// rows row0.. of out[., col0 .. col0 + 63] (below col_end) from the turned piece
__device__ __forceinline__ void turn_write_bf16(const float* turn, int lane, bf16* out, long ldo, int row0, int T,
                                                int col0, int col_end, bool aligned) {
    const int sub = lane >> 3, col = col0 + (lane & 7) * 8;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const int row = row0 + 4 * p + sub;
        const uint4 v = *reinterpret_cast<const uint4*>(turn + (4 * p + sub) * TURN_LD + (lane & 7) * 4);
        if (row >= T || col >= col_end) continue;
        bf16* dst = out + (size_t)row * ldo + col;
        if (aligned && col + 8 <= col_end) {
            *reinterpret_cast<uint4*>(dst) = v;
        } else {
            const bf16* e = reinterpret_cast<const bf16*>(&v);
            for (int i = 0; i < 8; ++i)
                if (col + i < col_end) dst[i] = e[i];
        }
    }
}
// the same for 32 fp32 columns; ADD: out += piece, `old` holding out's values where `vec` (read before)
template <bool ADD>
__device__ __forceinline__ void turn_write_f32(const float* turn, int lane, float* out, long ldo, int row0, int T,
                                               int col0, int col_end, bool vec, const float4* old) {
    const int sub = lane >> 3, col = col0 + (lane & 7) * 4;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const int row = row0 + 4 * p + sub;
        const float4 d = *reinterpret_cast<const float4*>(turn + (4 * p + sub) * TURN_LD + (lane & 7) * 4);
        if (row >= T) continue;
        float* dst = out + (size_t)row * ldo + col;
        if (vec) {
            *reinterpret_cast<float4*>(dst) = ADD ? make_float4(old[p].x + d.x, old[p].y + d.y, old[p].z + d.z, old[p].w + d.w) : d;
        } else {
            const float dd[4] = {d.x, d.y, d.z, d.w};
            for (int i = 0; i < 4; ++i)
                if (col + i < col_end) dst[i] = ADD ? dst[i] + dd[i] : dd[i];
        }
    }
}

// TWO: a stage holds two 64-column tiles of K per operand, each operand's brought in by one copy (pairs always;
// single CTAs on 128-column tiles where K is a multiple of 64: three stages of 64 KB instead of six of 32 KB)
template <int BN, int EPI, typename OutT, bool PAIR, bool TWO = PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    OutT* __restrict__ out, int T, int F, int K, long ldo, int m_tiles, int n_tiles,
                    int* __restrict__ status, int k_splits, int kb_per_split, size_t split_stride,
                    float* parts, int* flags, const __grid_constant__ CUtensorMap map_out, int out_by_copies) {
    static_assert(!PAIR || BN == 256 || BN == 192, "a pair works on tiles of 256 tokens x 256 or 192 features");
    static_assert(!PAIR || TWO, "pairs take two tiles of K per stage");
    static_assert(PAIR || !TWO || BN == 128, "single CTAs take two tiles of K per stage on 128-column tiles only");
    constexpr int STAGES = PAIR ? pair_stages() : TWO ? stages_of(BN) / 2 : stages_of(BN);
    constexpr int W_ROWS = PAIR ? BN / 2 : BN;                           // weight rows that this CTA loads per K block
    // Pairs take two tiles of 64 columns of K per stage, each operand's in one copy (see make_map): with one tile
    // per copy the copies took longer than the MMAs (0.31 us per stage of 32 KB against 0.27 us).
    constexpr int SLABS = TWO ? PAIR_SLABS : 1;
    constexpr uint32_t X_BYTES = BM * BK * 2 * SLABS, W_BYTES = W_ROWS * BK * 2 * SLABS;
    constexpr uint32_t TMEM_COLS = 2 * BN > 256 ? 512 : 2 * BN;          // two accumulators (a power of two of columns)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t x_smem = base, w_smem = base + STAGES * X_BYTES;
    const uint32_t epi_smem = w_smem + STAGES * W_BYTES;                 // 1,024-byte aligned: the ring's sizes are
    const uint32_t bars = epi_smem + (uint32_t)epilogue_smem(EPI);
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, acc_full0 = bars + 16 * STAGES,
                   acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (acc_empty0 + 16 - raw));
    float* turn_base = reinterpret_cast<float*>(smem_raw + (epi_smem - raw));
    __shared__ int s_abort, s_parts_missing;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + BK * SLABS - 1) / (BK * SLABS);                // stages of K
    const uint32_t rank = PAIR ? cluster_rank() : 0u;                    // rank 0 of a pair issues the MMAs
    constexpr int TILE_M = PAIR ? 2 * BM : BM;
    constexpr int GROUP = PAIR ? 2 : 1;                                  // CTAs that work on a piece together
    const int group_no = blockIdx.x / GROUP, n_groups = gridDim.x / GROUP;
    const bool stream = STREAM_BUILD && parts != nullptr;
    Walk walk0;
    walk0.stream = stream;
    walk0.n_kb = n_kb;
    walk0.n_tiles_mn = m_tiles * n_tiles;                                // PAIR: tiles of 256 tokens
    walk0.kb_per_split = kb_per_split;
    walk0.unit = group_no;
    walk0.unit_step = n_groups;
    walk0.unit_end = walk0.n_tiles_mn * k_splits;
    const long total_kb = (long)walk0.n_tiles_mn * n_kb;
    walk0.pos = stream ? stream_begin(total_kb, n_groups, group_no) : 0;
    walk0.hi = stream ? stream_begin(total_kb, n_groups, group_no + 1) : 0;

    if (threadIdx.x == 0) {
        WIDE_TRACE(0);
        s_abort = 0;
        s_parts_missing = 0;
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
#ifdef PLM_WIDE_TRACE
            long long waited_empty = 0, p_begin = clock64();
#endif
            int it = 0;                                                  // K blocks issued so far, over all pieces
            bool ok = true;
            Walk walk = walk0;
            Piece w;
            while (ok && walk.next(w)) {
                const int m0 = (w.tile % m_tiles) * TILE_M + (int)rank * BM, f0 = (w.tile / m_tiles) * BN + (int)rank * W_ROWS;
                // The stream walk takes a tile's K blocks in a turned order (a sum in any order), chosen so that
                // all CTAs are at the same few places of K at the same time, as CTAs that walk whole tiles are:
                // what one SM asks the L2 for, others ask for too.  A tile cut between CTAs starts where its
                // first cut is (the CTA that starts there is at its own first step); a whole tile starts at the
                // step that its CTA is at.
                int turn_k = 0;
                if (stream) {
                    if (w.kind == PIECE_WHOLE) {
                        turn_k = it % n_kb;
                    } else {
                        long cut = walk0.hi;                             // an owner's tile is cut where its range ends
                        if (w.kind == PIECE_PART) {
                            int c = group_no;
                            while (c > 0 && stream_begin(total_kb, n_groups, c - 1) > w.tile_end - n_kb) --c;
                            cut = stream_begin(total_kb, n_groups, c);
                        }
                        turn_k = (int)((w.tile_end - cut) % n_kb);       // n_kb - (cut - the tile's first block)
                    }
                }
                for (int kb0 = w.kb_begin; kb0 < w.kb_end; ++kb0, ++it) {
                    const int kb = kb0 + turn_k < n_kb ? kb0 + turn_k : kb0 + turn_k - n_kb;
                    const int s = it % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    WIDE_TRACE_CLOCK(e0);
                    if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, status, 1)) { s_abort = 1; ok = false; break; }
#ifdef PLM_WIDE_TRACE
                    waited_empty += clock64() - e0;                      // cycles this thread waited for a free stage
#endif
                    if (PAIR) {
                        // both CTAs' tiles count at the "full" barrier of rank 0, which expects them all
                        const uint32_t full = cluster_map_addr(full0 + 8 * s, 0);
                        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * (X_BYTES + W_BYTES));
                        tma_load_3d_pair(w_smem + s * W_BYTES, &map_w, full, f0, kb * SLABS);
                        if (!waited) { pdl_wait(); waited = true; }
                        tma_load_3d_pair(x_smem + s * X_BYTES, &map_x, full, m0, kb * SLABS);
                    } else {
                        mbar_expect_tx(full0 + 8 * s, X_BYTES + W_BYTES);
                        // weights are written by no kernel of the step: they may be requested at once
                        if (TWO) tma_load_3d(w_smem + s * W_BYTES, &map_w, full0 + 8 * s, f0, kb * SLABS);
                        else tma_load_2d(w_smem + s * W_BYTES, &map_w, full0 + 8 * s, kb * BK, f0);
                        if (!waited) { pdl_wait(); waited = true; WIDE_TRACE(1); }   // activations come from the kernel before
                        if (TWO) tma_load_3d(x_smem + s * X_BYTES, &map_x, full0 + 8 * s, m0, kb * SLABS);
                        else tma_load_2d(x_smem + s * X_BYTES, &map_x, full0 + 8 * s, kb * BK, m0);
                    }
                }
            }
            WIDE_TRACE(2);
#ifdef PLM_WIDE_TRACE
            WIDE_TRACE_VALUE(7, (unsigned long long)waited_empty);       // of a CTA with one piece: points 7..10 are cycle counts
            WIDE_TRACE_VALUE(8, (unsigned long long)(clock64() - p_begin));
#endif
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
            Walk walk = walk0;
            Piece w;
#ifdef PLM_WIDE_TRACE
            long long waited_full = 0, m_begin = clock64();
#endif
            for (; ok && walk.next(w); ++j) {
                const int acc = j & 1;
                // the epilogue must have read this accumulator's previous piece out
                if (!mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, status, 2)) { s_abort = 1; ok = false; break; }
                tc_fence_after();
                for (int kb = w.kb_begin; kb < w.kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    WIDE_TRACE_CLOCK(f0_);
                    if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, status, 2)) { s_abort = 1; ok = false; break; }
#ifdef PLM_WIDE_TRACE
                    waited_full += clock64() - f0_;                      // cycles this thread waited for loads to land
#endif
                    tc_fence_after();
                    const uint64_t xd = smem_desc_sw128(x_smem + s * X_BYTES);
                    const uint64_t wd = smem_desc_sw128(w_smem + s * W_BYTES);
#ifndef PLM_WIDE_LOADS_ONLY                                              // a measuring build: what the copies alone take
#pragma unroll
                    for (int k = 0; k < SLABS * (BK / UMMA_K); ++k) {
                        // a stage holds SLABS tiles of 64 columns of K one behind the other
                        const uint64_t x_off = (uint64_t)(((k / (BK / UMMA_K)) * (BM * BK * 2) + (k % (BK / UMMA_K)) * UMMA_K * 2) / 16);
                        const uint64_t w_off = (uint64_t)(((k / (BK / UMMA_K)) * (W_ROWS * BK * 2) + (k % (BK / UMMA_K)) * UMMA_K * 2) / 16);
                        if (PAIR)
                            tc_mma_bf16_pair(tmem_base + acc * BN, xd + x_off, wd + w_off, idesc, (kb > w.kb_begin || k > 0) ? 1u : 0u);
                        else
                            tc_mma_bf16(tmem_base + acc * BN, xd + x_off, wd + w_off, idesc, (kb > w.kb_begin || k > 0) ? 1u : 0u);
                    }
#endif
                    if (PAIR) tc_commit_pair(empty0 + 8 * s); else tc_commit(empty0 + 8 * s);
                }
                if (PAIR) tc_commit_pair(acc_full0 + 8 * acc); else tc_commit(acc_full0 + 8 * acc);
            }
            WIDE_TRACE(3);
#ifdef PLM_WIDE_TRACE
            WIDE_TRACE_VALUE(9, (unsigned long long)waited_full);
            WIDE_TRACE_VALUE(10, (unsigned long long)(clock64() - m_begin));
#endif
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        float* turn = turn_base + quarter * 32 * TURN_LD;
        const int my_row = quarter * 32 + lane;                          // the row of the tile that this thread holds
        pdl_wait();                                                      // the output may still be in use by an earlier kernel
        int j = 0;
        bool ok = true;
        Walk walk = walk0;
        Piece w;
        for (; ok && walk.next(w); ++j) {
            const int acc = j & 1;
            const int m0 = (w.tile % m_tiles) * TILE_M + (int)rank * BM, f0 = (w.tile / m_tiles) * BN;
            const int row0 = m0 + quarter * 32;                          // this warp's 32 token rows
            const uint32_t tacc = tmem_base + lane_bits + acc * BN;
            // an owner's tile: the parts that the CTAs after this one left, once their flags are up (they are
            // long before this CTA gets here: a part is the first thing its CTA does)
            int n_parts = 0;
            if (STREAM_BUILD && w.kind == PIECE_OWNER) {
                while (group_no + 1 + n_parts < n_groups &&
                       stream_begin(total_kb, n_groups, group_no + 1 + n_parts) < w.tile_end) ++n_parts;
                for (int p = 0; p < n_parts; ++p) {
                    bool up = false;
                    for (uint32_t i = 0; i < WAIT_LIMIT / 8 && !up; ++i) up = ld_acquire(flags + blockIdx.x + GROUP * (1 + p)) != 0;
                    if (!up) { if (status) atomicCAS(status, 0, 4); s_parts_missing = 1; }
                }
                epilogue_sync();                                         // all four warps take the same way from here
                if (s_parts_missing) { s_abort = 1; ok = false; n_parts = 0; }
            }
            // the first of the parts: the slot of the CTA of this rank in the next group (a pair: each CTA its 128 rows)
            const float* theirs = parts + (size_t)(blockIdx.x + GROUP) * BM * BN;
            // What the piece's first columns need from memory is asked for before the accumulator is waited
            // for, and every further 32 columns' while the 32 before them are written: one trip to the L2 per
            // 32 columns would otherwise stand between the last MMA and the end of the kernel.
            constexpr bool F32_OUT = EPI != EPI_SWIGLU && sizeof(OutT) == 4;
            float* outf = reinterpret_cast<float*>(out) + (size_t)w.ks * split_stride;
            const bool aligned4 = (ldo % 4 == 0) && ((uintptr_t)outf % 16 == 0);
            const int sub = lane >> 3, col4 = (lane & 7) * 4;            // pass p: row 4 p + sub, four columns from col4
            float4 old_n[8], part_n[8];
            auto get_old = [&](int c) {
                if (EPI == EPI_RESIDUAL && aligned4 && f0 + c + 32 <= F) {
#pragma unroll
                    for (int p = 0; p < 8; ++p) {
                        const int row = row0 + 4 * p + sub;
                        old_n[p] = row < T ? *reinterpret_cast<const float4*>(outf + (size_t)row * ldo + f0 + c + col4)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            };
            auto get_part = [&](int c) {
                if (STREAM_BUILD && n_parts > 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        part_n[i] = __ldcg(reinterpret_cast<const float4*>(theirs + part_offset(my_row, c + 4 * i)));
                }
            };
            // r += the parts' columns c .. c + 31: the first part from `first` (asked for earlier), the others now
            auto add_parts = [&](uint32_t* r, int c, const float4* first) {
                if (!STREAM_BUILD) return;
                if (n_parts > 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + first[i].x);
                        r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + first[i].y);
                        r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + first[i].z);
                        r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + first[i].w);
                    }
                }
                for (int p = 1; p < n_parts; ++p) {
                    const float* more = theirs + (size_t)p * GROUP * BM * BN;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(more + part_offset(my_row, c + 4 * i)));
                        r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + a.x);
                        r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + a.y);
                        r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + a.z);
                        r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + a.w);
                    }
                }
            };
            if (w.kind != PIECE_PART && EPI != EPI_SWIGLU) {
                if (F32_OUT && !out_by_copies) get_old(0);
                get_part(0);
            }
            if (threadIdx.x == 64) WIDE_TRACE(4 + 3 * j);
            const bool ready = mbar_wait(acc_full0 + 8 * acc, (j >> 1) & 1, status, 3);
            tc_fence_after();
            if (threadIdx.x == 64) WIDE_TRACE(5 + 3 * j);
            if (!ready) {
                s_abort = 1;
                ok = false;
            } else if (STREAM_BUILD && w.kind == PIECE_PART) {
                float* mine = parts + (size_t)blockIdx.x * BM * BN;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tc_ld32(tacc + c, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4*>(mine + part_offset(my_row, c + i)) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
                }
                __threadfence();
            } else if (EPI == EPI_SWIGLU) {
                bf16* outb = reinterpret_cast<bf16*>(out);
                const bool aligned = (ldo % 8 == 0) && ((uintptr_t)outb % 16 == 0);
#pragma unroll 1
                for (int gq = 0; gq < BN; gq += 128) {
                    if (f0 + gq >= F) break;
#pragma unroll 1
                    for (int cc = 0; cc < 64; cc += 32) {
                        uint32_t gt[32], up[32];
                        tc_ld32(tacc + gq + cc, gt);
                        tc_ld32(tacc + gq + 64 + cc, up);
                        tc_wait_ld();
                        for (int p = 0; STREAM_BUILD && p < n_parts; ++p) {
                            const float* more = theirs + (size_t)p * GROUP * BM * BN;
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                const float4 a = __ldcg(reinterpret_cast<const float4*>(more + part_offset(my_row, gq + cc + i)));
                                const float4 b = __ldcg(reinterpret_cast<const float4*>(more + part_offset(my_row, gq + 64 + cc + i)));
                                gt[i] = __float_as_uint(__uint_as_float(gt[i]) + a.x); gt[i + 1] = __float_as_uint(__uint_as_float(gt[i + 1]) + a.y);
                                gt[i + 2] = __float_as_uint(__uint_as_float(gt[i + 2]) + a.z); gt[i + 3] = __float_as_uint(__uint_as_float(gt[i + 3]) + a.w);
                                up[i] = __float_as_uint(__uint_as_float(up[i]) + b.x); up[i + 1] = __float_as_uint(__uint_as_float(up[i + 1]) + b.y);
                                up[i + 2] = __float_as_uint(__uint_as_float(up[i + 2]) + b.z); up[i + 3] = __float_as_uint(__uint_as_float(up[i + 3]) + b.w);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            gt[i] = __float_as_uint(swiglu_bf16(__uint_as_float(gt[i]), __uint_as_float(up[i])));
                        if (out_by_copies) {
                            const uint32_t piece = epi_smem + (uint32_t)(((gq >> 7) & 1) * OUT_PIECE);
                            if (cc == 0) {
                                if (threadIdx.x == 64) copies_have_read<1>();    // the copy that read this piece's room before
                                epilogue_sync();
                            }
                            stage_bf16(smem_raw + (piece - raw), my_row, cc >> 3, gt);
                        } else {
                            turn_put_bf16(turn, lane, cc >> 5, gt);
                        }
                    }
                    if (out_by_copies) {
                        fence_for_copies();
                        epilogue_sync();
                        if (threadIdx.x == 64)
                            copy_store_out(&map_out, epi_smem + (uint32_t)(((gq >> 7) & 1) * OUT_PIECE), (f0 + gq) / 2, m0);
                    } else {
                        __syncwarp();
                        turn_write_bf16(turn, lane, outb, ldo, row0, T, (f0 + gq) / 2, F / 2, aligned);
                        __syncwarp();                                    // the piece is read before the next one overwrites it
                    }
                }
            } else {
                // 32 columns at a time, two register sets in turn: the next 32 columns are on their way out of
                // the tensor memory while these are converted, turned and written
                bf16* outb = reinterpret_cast<bf16*>(out);
                const bool aligned8 = (ldo % 8 == 0) && ((uintptr_t)outb % 16 == 0);
                const int c_end = min(BN, (F - f0 + 63) & ~63);
                auto piece32 = [&](uint32_t* r, int c) {
                    float4 old[8], part[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) { old[i] = old_n[i]; part[i] = part_n[i]; }
                    if (c + 32 < c_end) {
                        if (F32_OUT && !out_by_copies) get_old(c + 32);
                        get_part(c + 32);
                    }
                    add_parts(r, c, part);
                    if (EPI == EPI_RESIDUAL && out_by_copies) {
                        // the piece goes to shared memory as the copy engine wants it (a row's eight 16-byte chunks
                        // at places turned by the row's number), and one thread hands it over; two pieces in turn
                        const uint32_t piece = epi_smem + (uint32_t)(((c >> 5) & 1) * OUT_PIECE);
                        if (threadIdx.x == 64) copies_have_read<1>();        // the copy that read this piece's room before
                        epilogue_sync();
                        uint8_t* mine = smem_raw + (piece - raw) + my_row * 128;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<uint4*>(mine + ((i ^ (my_row & 7)) << 4)) =
                                make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                        fence_for_copies();
                        epilogue_sync();
                        if (threadIdx.x == 64 && f0 + c < F) copy_add_out(&map_out, piece, f0 + c, m0);
                    } else if (F32_OUT && out_by_copies) {               // a plain store of floats, the same way
                        const uint32_t piece = epi_smem + (uint32_t)(((c >> 5) & 1) * OUT_PIECE);
                        if (threadIdx.x == 64) copies_have_read<1>();
                        epilogue_sync();
                        uint8_t* mine = smem_raw + (piece - raw) + my_row * 128;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<uint4*>(mine + ((i ^ (my_row & 7)) << 4)) =
                                make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                        fence_for_copies();
                        epilogue_sync();
                        if (threadIdx.x == 64 && f0 + c < F) copy_store_out(&map_out, piece, f0 + c, m0);
                    } else if (!F32_OUT && out_by_copies) {              // bf16: two rounds of 32 columns fill a piece of 64
                        const uint32_t piece = epi_smem + (uint32_t)(((c >> 6) & 1) * OUT_PIECE);
                        if (!(c & 32)) {
                            if (threadIdx.x == 64) copies_have_read<1>();
                            epilogue_sync();
                        }
                        stage_bf16(smem_raw + (piece - raw), my_row, (c & 32) >> 3, r);
                        if (c & 32) {
                            fence_for_copies();
                            epilogue_sync();
                            if (threadIdx.x == 64 && f0 + (c & ~63) < F) copy_store_out(&map_out, piece, f0 + (c & ~63), m0);
                        }
                    } else if (F32_OUT) {
                        if (f0 + c < F) {
                            turn_put_f32(turn, lane, r);
                            __syncwarp();
                            turn_write_f32<EPI == EPI_RESIDUAL>(turn, lane, outf, ldo, row0, T, f0 + c, F,
                                                                aligned4 && (f0 + c + 32 <= F), old);
                            __syncwarp();                                // the piece is read before the next one overwrites it
                        }
                    } else {
                        turn_put_bf16(turn, lane, (c >> 5) & 1, r);      // two rounds fill a turned piece of 64 columns
                        if (c & 32) {
                            __syncwarp();
                            turn_write_bf16(turn, lane, outb, ldo, row0, T, f0 + (c & ~63), F, aligned8);
                            __syncwarp();
                        }
                    }
                };
                uint32_t ra[32], rb[32];
                tc_ld32(tacc, ra);
#pragma unroll 1
                for (int c = 0; c < c_end; c += 64) {
                    tc_wait_ld_into(ra);
                    if (threadIdx.x == 64 && j == 0 && c == 0) WIDE_TRACE(13);
                    tc_ld32(tacc + c + 32, rb);
                    piece32(ra, c);
                    if (threadIdx.x == 64 && j == 0 && c == 0) WIDE_TRACE(14);
                    tc_wait_ld_into(rb);
                    if (c + 64 < c_end) tc_ld32(tacc + c + 64, ra);
                    piece32(rb, c + 32);
                    if (threadIdx.x == 64 && j == 0 && c == 0) WIDE_TRACE(15);
                }
            }
            if (STREAM_BUILD && w.kind == PIECE_PART) {                  // all of the part is written: the flag goes up
                epilogue_sync();
                if (threadIdx.x == 64 && ready) st_release(flags + blockIdx.x, 1);
            }
            if (STREAM_BUILD && n_parts > 0) {                           // the flags go down for the next launch
                epilogue_sync();
                if (threadIdx.x == 64)
                    for (int p = 0; p < n_parts; ++p) flags[blockIdx.x + GROUP * (1 + p)] = 0;
            }
            if (!ready) break;
            if (threadIdx.x == 64) WIDE_TRACE(6 + 3 * j);
            tc_fence_before();
            // this accumulator may be overwritten (a pair: says so to rank 0, which issues the MMAs)
            if (PAIR) mbar_arrive_cluster(cluster_map_addr(acc_empty0 + 8 * acc, 0)); else mbar_arrive(acc_empty0 + 8 * acc);
        }
    }
    if (threadIdx.x == 64) copies_done();                                // this thread's copies out of shared memory
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

// The result as the copy engine writes it (or adds to it): pieces of 128 rows x 128 bytes, 128-byte swizzle.
// `usable`: whether it can (16-byte aligned rows); else the epilogue's threads write by themselves.
struct OutMap { CUtensorMap map; int usable; };
// `out` [T, F_out] with leading dimension ldo elements, of floats (pieces of 128 x 32) or bf16 (128 x 64).
OutMap out_map(const void* out, int out_is_f32, int T, int F_out, long ldo) {
    OutMap m;
    memset(&m, 0, sizeof(m));
    const int esize = out_is_f32 ? 4 : 2;
    if ((ldo * esize) % 16 || ((uintptr_t)out & 15)) return m;
    struct Entry { const void* ptr; int T, F, f32; long ldo; bool used; CUtensorMap map; };
    static Entry table[64];
    static std::mutex lock;
    Entry& e = table[(((size_t)out >> 8) * 0x9E3779B97F4A7C15ull >> 40) % 64];
    {
        std::lock_guard<std::mutex> g(lock);
        if (e.used && e.ptr == out && e.T == T && e.F == F_out && e.ldo == ldo && e.f32 == out_is_f32) {
            m.map = e.map;
            m.usable = 1;
            return m;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return m;
    cuuint64_t dims[2] = {(cuuint64_t)F_out, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)ldo * esize};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)BM};
    cuuint32_t estr[2] = {1, 1};
    if (fn(&m.map, out_is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(out),
           dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return m;
    m.usable = 1;
    std::lock_guard<std::mutex> g(lock);
    e.ptr = out; e.T = T; e.F = F_out; e.ldo = ldo; e.f32 = out_is_f32; e.map = m.map; e.used = true;
    return m;
}

// The width of a pair's tiles for (T, F): 256 features, or 192 where that needs less time over the 74 pairs (rounds
// of tiles x the tile's width: 3,072 features at 2,048 tokens are 96 tiles of 256, two rounds the second of which is
// a third full, or 128 tiles of 192, two rounds of three quarters of the work each).  SwiGLU keeps 256 (its tiles
// hold gate and up rows in groups of 128).
int pair_width(int T, int F, int epilogue) {
    if (epilogue == EPI_SWIGLU) return 256;
    const long m_tiles = (T + 2 * BM - 1) / (2 * BM), pairs = sm_count() / 2;
    const long r256 = (m_tiles * ((F + 255) / 256) + pairs - 1) / pairs, r192 = (m_tiles * ((F + 191) / 192) + pairs - 1) / pairs;
    return r192 * 192 < r256 * 256 ? 192 : 256;
}

template <int BN, int EPI, typename OutT>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, OutT* out, int T, int F, int K, long ldo, int* status,
                cudaStream_t stream, float* parts = nullptr, int* flags = nullptr, int streamed_pairs = 0) {
    static bool configured = false;
    constexpr size_t smem = pair_smem(EPI);
    auto kern = gemm_tc_wide_kernel<BN, EPI, OutT, true>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = (T + 2 * BM - 1) / (2 * BM), n_tiles = (F + BN - 1) / BN;
    int pairs = sm_count() / 2;
    if (m_tiles * n_tiles < pairs) pairs = m_tiles * n_tiles;
    if (streamed_pairs) pairs = streamed_pairs;
    const OutMap mo = out_map(out, sizeof(OutT) == 4, T, EPI == EPI_SWIGLU ? F / 2 : F, ldo);
    return plm_status_of(launch_pdl_cluster(kern, dim3(2 * pairs), dim3(NUM_THREADS), dim3(2, 1, 1), smem, stream, mx, mw,
                                            out, T, F, K, ldo, m_tiles, n_tiles, status, 1,
                                            (K + BK * PAIR_SLABS - 1) / (BK * PAIR_SLABS), (size_t)0,
                                            streamed_pairs ? parts : (float*)nullptr, streamed_pairs ? flags : (int*)nullptr,
                                            mo.map, mo.usable));
}

// The parts and flags of the stream walk (see Walk): `slots` slots of BM * 256 floats and as many flags, which
// are zero between launches.  nullptr: whole tiles only.
struct StreamSpace { float* parts; int* flags; int slots; };

// How many CTAs walk the K blocks of all tiles as one stream; 0: the tiles are handed out whole (they fill
// the SMs' rounds well enough, or there is no workspace).
// `group`: 1 for single CTAs, 2 for pairs (the answer then counts pairs); `n_kb` counts stages of `slabs` tiles of K.
int stream_ctas(int tiles, int n_kb, const StreamSpace& space, int group = 1, int slabs = 1) {
    if (!space.parts || !space.flags) return 0;
    const int sms = sm_count() / group;
    int ctas = sms < space.slots / group ? sms : space.slots / group;
    const long total = (long)tiles * n_kb;
    const int least = 8 / slabs;                                         // at least 8 tiles of K each
    if (total / least < ctas) ctas = (int)(total / least);
    if (ctas > 2 * tiles) ctas = 2 * tiles;                              // a tile is cut among three CTAs at most: its owner adds the parts up alone
    if (ctas < 2) return 0;
    // Only where the tiles do not fill one round over the SMs.  With more tiles the stream was measured slower than
    // whole tiles although it leaves no SM idle (4,096 x 2,048 x 8,192 by pairs: 110 against 105 us; 1,024 x 16,384 x
    // 2,048 with SwiGLU: 59 against 50 us): under the power cap the SMs that still work in a ragged last round run
    // at a higher clock, and the parts cost what they cost.
    if (tiles >= sms) return 0;
    // In K blocks of time: a round of whole tiles takes a tile's K blocks; the stream takes total / ctas and what
    // its parts cost: some CTA's only piece is a part that is ready when everything else is, and its owner's
    // epilogue comes after that part's: measured at about 30 blocks' time.
    const long whole = n_kb, streamed = (total + ctas - 1) / ctas + 32 / slabs;
    return streamed < whole ? ctas : 0;
}

template <int BN, int EPI, typename OutT, bool TWO = false>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, OutT* out, int T, int F, int K, long ldo, int* status,
           cudaStream_t stream, int k_splits = 1, int kb_per_split = 0, size_t split_stride = 0,
           StreamSpace space = StreamSpace{nullptr, nullptr, 0}, int streamed = 0) {
    static bool configured = false;
    constexpr size_t smem = wide_smem(BN, EPI);
    auto kern = gemm_tc_wide_kernel<BN, EPI, OutT, false, TWO>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = (T + BM - 1) / BM, n_tiles = (F + BN - 1) / BN;
    const int units = m_tiles * n_tiles * k_splits;
    int ctas = units < sm_count() ? units : sm_count();
    if (kb_per_split <= 0) kb_per_split = (K + BK * (TWO ? 2 : 1) - 1) / (BK * (TWO ? 2 : 1));
    if (k_splits > 1) streamed = 0;
    if (streamed) ctas = streamed;
    // (the slices of a K split go to scratch memory by the threads' own stores)
    OutMap mo = out_map(out, sizeof(OutT) == 4, T, EPI == EPI_SWIGLU ? F / 2 : F, ldo);
    if (k_splits > 1) mo.usable = 0;
    return plm_status_of(launch_pdl(kern, dim3(ctas), dim3(NUM_THREADS), smem, stream, mx, mw, out, T, F, K, ldo, m_tiles,
                                    n_tiles, status, k_splits, kb_per_split, split_stride,
                                    streamed ? space.parts : (float*)nullptr, streamed ? space.flags : (int*)nullptr,
                                    mo.map, mo.usable));
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

// How the single-CTA form runs (T, F, K): the tile width, the parts of K that pass through scratch memory
// (store epilogue only), and the CTAs of the stream walk (0: whole tiles).
struct Plan { int bn, k_splits, kb_per, streamed, slabs; };    // kb_per: stages of `slabs` tiles of K per part
Plan wide_plan(int T, int F, int K, int epilogue, const StreamSpace& space) {
    Plan p{128, 1, 0, 0, 1};
    const long m_tiles = (T + BM - 1) / BM, sms = sm_count();
    const bool may_be_wide = F >= 2048 && T >= 256;
    if (may_be_wide) {
        // 256 columns feed the tensor cores best (a 128-column tile takes 0.8 of a 256-column tile's time for
        // half the work), but CTAs that walk whole tiles finish earlier with narrow tiles where those need no
        // more rounds over the SMs than the wide ones (prompts of a few hundred tokens).
        const long wide = (m_tiles * ((F + 255) / 256) + sms - 1) / sms, narrow = (m_tiles * ((F + 127) / 128) + sms - 1) / sms;
        p.bn = 0.8 * (double)narrow < (double)wide ? 128 : 256;
    }
    // 128-column tiles take two tiles of K per stage and copy where K allows it (see the kernel's TWO)
    p.slabs = (p.bn == 128 && K % BK == 0) ? PAIR_SLABS : 1;
    int n_kb = (K + BK * p.slabs - 1) / (BK * p.slabs);                  // stages of K
    p.kb_per = n_kb;
    const long tiles = m_tiles * ((F + p.bn - 1) / p.bn);
    // K splits where the tiles leave at least half of the SMs without work and K is long enough to cut
    if (epilogue == EPI_STORE && tiles * 2 <= sms && F % 4 == 0) {
        int splits = (int)(sms / tiles);
        if (splits > 8) splits = 8;
        if (splits > n_kb * p.slabs / 4) splits = n_kb * p.slabs / 4;    // at least four tiles of K a part
        if (splits < 1) splits = 1;
        p.kb_per = (n_kb + splits - 1) / splits;
        p.k_splits = (n_kb + p.kb_per - 1) / p.kb_per;                     // no part of K is empty
    }
    if (p.k_splits > 1) return p;
    // The stream walk fills the SMs whatever the number of tiles: with wide tiles where it pays at all.
    if (may_be_wide && p.bn != 256) {
        const int n_kb1 = (K + BK - 1) / BK;
        const int streamed = stream_ctas((int)(m_tiles * ((F + 255) / 256)), n_kb1, space);
        if (streamed) { p.bn = 256; p.slabs = 1; p.kb_per = n_kb1; p.streamed = streamed; return p; }
    }
    p.streamed = stream_ctas((int)tiles, n_kb, space, 1, p.slabs);
    return p;
}

bool operands_ok(const void* x, const void* w, int K, long ldx, long ldw) {
    return K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((((uintptr_t)x | (uintptr_t)w) & 15) == 0);
}

}  // namespace

// Into how many parts plm_gemm_tc_wide cuts K for (T, F, K) with the store epilogue: it needs that many
// slices of T * F floats of scratch memory if the answer is more than 1.
extern "C" int plm_gemm_tc_wide_splits(int T, int F, int K) {
    return wide_plan(T, F, K, EPI_STORE, StreamSpace{nullptr, nullptr, 0}).k_splits;
}

// Floats of a slot of the stream walk's workspace (`parts` of plm_gemm_tc_wide_space holds `slots` of them).
extern "C" int plm_gemm_tc_wide_slot_floats() { return BM * 256; }

// out[T, F'] = epilogue(x[T, K] * w[F, K]^T), T > 64, bf16 operands that TMA can address (K and the
// leading dimensions multiples of 8, pointers 16-byte aligned).  epilogue 0: F' = F, out float32
// (out_dtype 0) or bfloat16 (1).  epilogue 1 (SwiGLU): w holds tiles of 64 gate rows followed by their
// 64 up rows (F a multiple of 128), F' = F / 2, out bfloat16.  epilogue 2: out += product, out float32.
// `scratch`: plm_gemm_tc_wide_splits(T, F, K) slices of T * F floats where that is more than 1 (else unused;
// without it K is not cut; epilogue 0 only).  `parts`, `flags`, `slots`: the workspace of the stream walk,
// `slots` * plm_gemm_tc_wide_slot_floats() floats and `slots` ints that are zero before the first launch and
// that launches of one stream at a time use (they leave them zero); nullptr: tiles are handed out whole.
extern "C" int plm_gemm_tc_wide_space(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                      int K, long ldx, long ldw, long ldo, float* scratch, float* parts, int* flags,
                                      int slots, int* status, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (!operands_ok(x, w, K, ldx, ldw)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && (F % 128 || out_dtype != PLM_BF16)) return PLM_ERR_SHAPE;
    if (epilogue == EPI_RESIDUAL && out_dtype != PLM_F32) return PLM_ERR_DTYPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU && epilogue != EPI_RESIDUAL) return PLM_ERR_UNSUPPORTED;
    if (out_dtype != PLM_F32 && out_dtype != PLM_BF16) return PLM_ERR_DTYPE;
    if (!STREAM_BUILD) parts = nullptr;                                  // this build walks whole tiles only
    const StreamSpace space{parts, flags, (parts && flags) ? slots : 0};
    const Plan plan = wide_plan(T, F, K, epilogue, space);
    const int bn = plan.bn, st = plan.streamed;
    const bool two = plan.slabs == 2;
    const bool cut = plan.k_splits > 1 && scratch && ldo == F && (((uintptr_t)scratch | (uintptr_t)out) & 15) == 0;
    const int k_splits = cut ? plan.k_splits : 1, kb_per = cut ? plan.kb_per : 0;
    CUtensorMap mx, mw;
    int rc;
    if ((rc = make_map(&mx, x, T, K, ldx, BM, plan.slabs)) != PLM_OK) return rc;
    if ((rc = make_map(&mw, w, F, K, ldw, bn, plan.slabs)) != PLM_OK) return rc;
// the kernel for this plan's tile width and stage, with the epilogue and result type given
#define PLM_WIDE_LAUNCH(EPI, OutT, outp, ld, splits, per, stride)                                                        \
    (bn == 256 ? launch<256, EPI, OutT, false>(mx, mw, outp, T, F, K, ld, status, stream, splits, per, stride, space, st)  \
     : two     ? launch<128, EPI, OutT, true>(mx, mw, outp, T, F, K, ld, status, stream, splits, per, stride, space, st)   \
               : launch<128, EPI, OutT, false>(mx, mw, outp, T, F, K, ld, status, stream, splits, per, stride, space, st))
    if (epilogue == EPI_SWIGLU) return PLM_WIDE_LAUNCH(EPI_SWIGLU, bf16, (bf16*)out, ldo, 1, 0, (size_t)0);
    if (epilogue == EPI_RESIDUAL) return PLM_WIDE_LAUNCH(EPI_RESIDUAL, float, (float*)out, ldo, 1, 0, (size_t)0);
    if (cut) {
        // the parts of K as units of work of their own, each into its slice of the scratch; then the sum
        const size_t stride = (size_t)T * F;
        rc = PLM_WIDE_LAUNCH(EPI_STORE, float, scratch, (long)F, k_splits, kb_per, stride);
        if (rc != PLM_OK) return rc;
        const size_t n4 = stride / 4;
        const int blocks = (int)((n4 + 255) / 256 < (size_t)(8 * sm_count()) ? (n4 + 255) / 256 : (size_t)(8 * sm_count()));
        if (out_dtype == PLM_F32)
            return plm_status_of(launch_pdl(reduce_splits_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                                            (const float*)scratch, (float*)out, k_splits, n4, stride));
        return plm_status_of(launch_pdl(reduce_splits_kernel<bf16>, dim3(blocks), dim3(256), 0, stream,
                                        (const float*)scratch, (bf16*)out, k_splits, n4, stride));
    }
    if (out_dtype == PLM_F32) return PLM_WIDE_LAUNCH(EPI_STORE, float, (float*)out, ldo, 1, 0, (size_t)0);
    return PLM_WIDE_LAUNCH(EPI_STORE, bf16, (bf16*)out, ldo, 1, 0, (size_t)0);
#undef PLM_WIDE_LAUNCH
}

// The same without any workspace: K is never cut and tiles are handed out whole.
extern "C" int plm_gemm_tc_wide(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                int K, long ldx, long ldw, long ldo, int* status, cudaStream_t stream) {
    return plm_gemm_tc_wide_space(x, w, out, out_dtype, epilogue, T, F, K, ldx, ldw, ldo, nullptr, nullptr, nullptr, 0,
                                  status, stream);
}

// How many pairs walk the stages of all 256 x 256 tiles as one stream for (T, F, K) with `slots` slots of workspace;
// 0: the pairs take whole tiles.
extern "C" int plm_gemm_tc_pair_streamed(int T, int F, int K, int slots) {
    float dummy_parts;
    int dummy_flags;
    if (slots <= 0 || K % BK) return 0;
    const StreamSpace space{&dummy_parts, &dummy_flags, slots};
    const int tiles = ((T + 2 * BM - 1) / (2 * BM)) * ((F + 255) / 256);
    return stream_ctas(tiles, (K + BK * PAIR_SLABS - 1) / (BK * PAIR_SLABS), space, 2, PAIR_SLABS);
}

// The same product by pairs of CTAs (tcgen05.mma.cta_group::2, tiles of 256 tokens x 256 features; see
// PAIR at the top).  For prompts of at least 256 tokens and at least 256 features.  `parts`, `flags`, `slots` as for
// plm_gemm_tc_wide_space: where the tiles are few, the pairs walk them as one stream.
extern "C" int plm_gemm_tc_pair_space(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                      int K, long ldx, long ldw, long ldo, float* parts, int* flags, int slots, int* status,
                                      cudaStream_t stream) {
    if (T <= 0 || F <= 0) return PLM_OK;
    if (!operands_ok(x, w, K, ldx, ldw)) return PLM_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU && (F % 128 || out_dtype != PLM_BF16)) return PLM_ERR_SHAPE;
    if (epilogue == EPI_RESIDUAL && out_dtype != PLM_F32) return PLM_ERR_DTYPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU && epilogue != EPI_RESIDUAL) return PLM_ERR_UNSUPPORTED;
    if (K % BK)          // the pairs' copies take whole tiles of 64 columns of K: other widths go to the single CTAs
        return plm_gemm_tc_wide_space(x, w, out, out_dtype, epilogue, T, F, K, ldx, ldw, ldo, nullptr, parts, flags, slots,
                                      status, stream);
    const int st = (STREAM_BUILD && parts && flags) ? plm_gemm_tc_pair_streamed(T, F, K, slots) : 0;
    const int bn = st ? 256 : pair_width(T, F, epilogue);                // (the stream walk's slots are for tiles of 256)
    CUtensorMap mx, mw;
    int rc;
    if ((rc = make_map(&mx, x, T, K, ldx, BM, PAIR_SLABS)) != PLM_OK) return rc;
    if ((rc = make_map(&mw, w, F, K, ldw, bn / 2, PAIR_SLABS)) != PLM_OK) return rc;
    if (epilogue == EPI_SWIGLU) return launch_pair<256, EPI_SWIGLU, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream, parts, flags, st);
    if (bn == 192) {
        if (epilogue == EPI_RESIDUAL) return launch_pair<192, EPI_RESIDUAL, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
        if (out_dtype == PLM_F32) return launch_pair<192, EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream);
        if (out_dtype == PLM_BF16) return launch_pair<192, EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream);
        return PLM_ERR_DTYPE;
    }
    if (epilogue == EPI_RESIDUAL) return launch_pair<256, EPI_RESIDUAL, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream, parts, flags, st);
    if (out_dtype == PLM_F32) return launch_pair<256, EPI_STORE, float>(mx, mw, (float*)out, T, F, K, ldo, status, stream, parts, flags, st);
    if (out_dtype == PLM_BF16) return launch_pair<256, EPI_STORE, bf16>(mx, mw, (bf16*)out, T, F, K, ldo, status, stream, parts, flags, st);
    return PLM_ERR_DTYPE;
}

// The same without a workspace: the pairs take whole tiles.
extern "C" int plm_gemm_tc_pair(const void* x, const void* w, void* out, int out_dtype, int epilogue, int T, int F,
                                int K, long ldx, long ldw, long ldo, int* status, cudaStream_t stream) {
    return plm_gemm_tc_pair_space(x, w, out, out_dtype, epilogue, T, F, K, ldx, ldw, ldo, nullptr, nullptr, 0, status, stream);
}

// For tests of the stream walk on the host: the pieces of CTA `cta` of `ctas` over `tiles` tiles of `n_kb` K
// blocks, four ints each (tile, first K block, end, kind: 0 whole, 1 part, 2 owner) into `out`, at most
// `max_pieces`; returns their number.
extern "C" int plm_gemm_tc_wide_pieces(int tiles, int n_kb, int ctas, int cta, int* out, int max_pieces) {
    Walk walk;
    walk.stream = true;
    walk.n_kb = n_kb;
    walk.n_tiles_mn = tiles;
    walk.kb_per_split = n_kb;
    walk.unit = walk.unit_end = walk.unit_step = 0;
    walk.pos = stream_begin((long)tiles * n_kb, ctas, cta);
    walk.hi = stream_begin((long)tiles * n_kb, ctas, cta + 1);
    Piece w;
    int n = 0;
    while (walk.next(w)) {
        if (n < max_pieces) { out[4 * n] = w.tile; out[4 * n + 1] = w.kb_begin; out[4 * n + 2] = w.kb_end; out[4 * n + 3] = w.kind; }
        ++n;
    }
    return n;
}

// How the single-CTA form runs (T, F, K) with `slots` slots of stream workspace (0: none): out[0] the tile
// width, out[1] the parts of K with scratch memory, out[2] the CTAs of the stream walk (0: whole tiles).
extern "C" int plm_gemm_tc_wide_how(int T, int F, int K, int epilogue, int slots, int* out) {
    float dummy_parts;
    int dummy_flags;
    const StreamSpace space{slots > 0 ? &dummy_parts : nullptr, slots > 0 ? &dummy_flags : nullptr, slots};
    const Plan p = wide_plan(T, F, K, epilogue, space);
    out[0] = p.bn;
    out[1] = p.k_splits;
    out[2] = p.k_splits == 1 ? p.streamed : 0;
    return PLM_OK;
}

#ifdef PLM_WIDE_TRACE
extern "C" int plm_gemm_tc_wide_trace_read(unsigned long long* host) {
    return plm_status_of(cudaMemcpyFromSymbol(host, plm_wide_trace, sizeof(unsigned long long) * 16 * PLM_SM_COUNT));
}
#endif
