// bfloat16 attention over the paged cache on the tensor cores (mma.sync
// m16n8k16, fp32 accumulation, fp32 softmax statistics), compiled for one head
// size: -DPLM_HD=<head_dim>, a multiple of 16 up to 256.
//
// For a query at position p, head h, KV head g = h / (H/G):
//   s_t = (q_h . K[t, g]) * scale for lo <= t <= p;  out_h = softmax(s) . V[:, g]
// with the running (max, sum, acc) recurrence of the reference's attn_core
// (picolm/model_attention.c:43-140) applied to 64 keys (prefill) or 16 keys
// (decode) at a time, and the reference's idea of serving all H/G query heads of
// a KV head from one pass over its keys (picolm/model_attention.c:142-150).
//
// Two kernels:
//   prefill  one CTA per (sequence, KV head, tile of 64 query rows); a row is a
//            (token, head-in-group) pair, so the heads of a group share every
//            K/V page that is loaded.  Causal, ragged over sequences.
//   decode   one CTA per (token, KV head x row group, split of the keys): the
//            splits' partial (max, sum, acc) go to a workspace and a small kernel
//            merges them with exp(m_i - m) weights, as the reference's split
//            kernel does (picolm/backend_gpu_kernels.cu:802, :911).
// K and V pages are [64 keys][HD] contiguous in the cache.  The prefill kernel copies them to shared
// memory with cp.async (rows padded by 16 bytes so that ldmatrix has no bank conflicts) in a multi-stage
// ring.  The decode kernel does the same for head sizes that are no multiple of 64; for those that are, one
// thread asks for whole pages by TMA (cp.async.bulk.tensor through a tensor map over the cache, 128-byte
// swizzle, an mbarrier per stage): unpadded tiles, one instruction per 8 KB instead of 512 copies of 16
// bytes, and ldmatrix addresses that undo the swizzle.
#include "tc_common.cuh"

#ifndef PLM_HD
#define PLM_HD 64
#endif

namespace {

constexpr int HD = PLM_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16 up to 256");
constexpr int LDS = HD + 8;                 // padded row length in elements
constexpr int TILE_ELEMS = 64 * LDS;        // one 64-row tile
constexpr int NT = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// 16 bytes if `full`, else zeros (the source is not read)
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool full) {
    const int n = full ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// A tile as TMA writes it with the 128-byte swizzle: HD / 64 parts of [64 rows][128 bytes], each 8 KB; within a
// part, the 16-byte chunk c of row r lies at chunk c ^ (r % 8).  `chunk` counts 16-byte chunks of the whole row.
constexpr bool HAS_TMA = HD % 64 == 0;
constexpr uint32_t SW_TILE_BYTES = 64 * HD * 2;
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * 8192 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Copy one page tile (64 rows of HD bf16, contiguous in global memory) into a padded smem tile.
// Rows at and beyond `valid` (places of the page that hold no key yet) are filled with zeros, so
// that whatever an earlier owner of the page left there cannot reach a sum.
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src, int valid) {
    constexpr int CPR = HD / 8;             // 16-byte chunks per row
    for (int c = threadIdx.x; c < 64 * CPR; c += NT) {
        const int row = c / CPR, col = c - row * CPR;
        cp_async16_zfill(smem_u32(dst + row * LDS + col * 8), src + row * HD + col * 8, row < valid);
    }
}

// S[16 x 8*NKT] += Q[16 x HD] . K^T for keys [key0, key0 + 8*NKT) of a tile; q_rows points at the
// warp's query rows in shared memory, of which this lane addresses row `arow` (lane % 16 where all 16
// rows are there; the decode kernel keeps fewer and points the others at a row of zeros).
template <int NKT>
__device__ __forceinline__ void qk_tile(float (&s)[NKT][4], const bf16* q_rows, const bf16* k_tile, int key0, int lane,
                                        int arow) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, smem_u32(q_rows + arow * LDS + ks * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int j = 0; j < NKT; j += 2) {
            uint32_t b[4];
            const int key = key0 + j * 8 + (lane & 7) + (lane >> 4) * 8;
            ldsm_x4(b, smem_u32(k_tile + key * LDS + ks * 16 + ((lane >> 3) & 1) * 8));
            mma_bf16(s[j], a, b[0], b[1]);
            mma_bf16(s[j + 1], a, b[2], b[3]);
        }
    }
}

// O[16 x HD] += P[16 x 8*NKT] . V for keys [key0, key0 + 8*NKT) of a tile; P comes from the score
// accumulators (already exponentiated), repacked as the A operand.
template <int NKT>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const float (&p)[NKT][4], const bf16* v_tile, int key0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NKT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
        a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
        a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
        a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
        const int key = key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int dt = 0; dt < HD / 8; dt += 2) {
            uint32_t b[4];
            ldsm_x4_t(b, smem_u32(v_tile + key * LDS + dt * 8 + (lane >> 4) * 8));
            mma_bf16(o[dt], a, b[0], b[1]);
            mma_bf16(o[dt + 1], a, b[2], b[3]);
        }
    }
}

// The same two products on a swizzled tile (shared-memory address `k_base` / `v_base`).
template <int NKT>
__device__ __forceinline__ void qk_tile_sw(float (&s)[NKT][4], const bf16* q_rows, uint32_t k_base, int key0, int lane,
                                           int arow) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, smem_u32(q_rows + arow * LDS + ks * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int j = 0; j < NKT; j += 2) {
            uint32_t b[4];
            const int key = key0 + j * 8 + (lane & 7) + (lane >> 4) * 8;
            ldsm_x4(b, k_base + sw_off(key, ks * 2 + ((lane >> 3) & 1)));
            mma_bf16(s[j], a, b[0], b[1]);
            mma_bf16(s[j + 1], a, b[2], b[3]);
        }
    }
}
template <int NKT>
__device__ __forceinline__ void pv_tile_sw(float (&o)[HD / 8][4], const float (&p)[NKT][4], uint32_t v_base, int key0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NKT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
        a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
        a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
        a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
        const int key = key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int dt = 0; dt < HD / 8; dt += 2) {
            uint32_t b[4];
            ldsm_x4_t(b, v_base + sw_off(key, dt + (lane >> 4)));
            mma_bf16(o[dt], a, b[0], b[1]);
            mma_bf16(o[dt + 1], a, b[2], b[3]);
        }
    }
}

// Scale, mask and fold one block of scores into the running softmax of the thread's two rows
// (row_lo = lane/4, row_hi = lane/4 + 8).  Scores become probabilities in place.
// key_base: position of the block's first key; pos_*: each row's own position (keys above it are
// masked); lo_*: first key each row may see.
template <int NKT>
__device__ __forceinline__ void softmax_block(float (&s)[NKT][4], float (&o)[HD / 8][4], float (&m)[2], float (&l)[2],
                                              float scale_log2, int key_base, int pos_lo, int pos_hi, int lo_lo,
                                              int lo_hi, int lane) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NKT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = key_base + j * 8 + (lane & 3) * 2 + (e & 1);
            const int hi = e >> 1;
            const bool ok = hi ? (key <= pos_hi && key >= lo_hi) : (key <= pos_lo && key >= lo_lo);
            const float v = ok ? s[j][e] * scale_log2 : -INFINITY;
            s[j][e] = v;
            mx[hi] = fmaxf(mx[hi], v);
        }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
        mx[hi] = fmaxf(mx[hi], __shfl_xor_sync(0xffffffffu, mx[hi], 1));
        mx[hi] = fmaxf(mx[hi], __shfl_xor_sync(0xffffffffu, mx[hi], 2));
        const float m_new = fmaxf(m[hi], mx[hi]);
        m_use[hi] = (m_new == -INFINITY) ? 0.f : m_new;         // a row that has seen no key yet
        alpha[hi] = exp2f(m[hi] - m_use[hi]);                    // m = -inf gives 0
        m[hi] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NKT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = exp2f(s[j][e] - m_use[e >> 1]);
            s[j][e] = p;
            sum[e >> 1] += p;
        }
    }
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
        sum[hi] += __shfl_xor_sync(0xffffffffu, sum[hi], 1);
        sum[hi] += __shfl_xor_sync(0xffffffffu, sum[hi], 2);
        l[hi] = l[hi] * alpha[hi] + sum[hi];
    }
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
        o[dt][0] *= alpha[0]; o[dt][1] *= alpha[0];
        o[dt][2] *= alpha[1]; o[dt][3] *= alpha[1];
    }
}

// ------------------------------------------------------------------- prefill
constexpr int PF_STAGES = 2;
constexpr size_t PF_SMEM = (size_t)(1 + 2 * PF_STAGES) * TILE_ELEMS * sizeof(bf16);

__global__ void __launch_bounds__(NT)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                    bf16* __restrict__ out, const int* __restrict__ seq_start, const int* __restrict__ seq_kv_len,
                    const int* __restrict__ block_table, int max_pages, int H, int G, float scale_log2, int window) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);
    bf16* k_s = q_s + TILE_ELEMS;                     // [PF_STAGES][64][LDS]
    bf16* v_s = k_s + PF_STAGES * TILE_ELEMS;
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z, g = blockIdx.y;
    const int R = H / G;
    const int t0 = seq_start[b], n_new = seq_start[b + 1] - t0;
    const int rows_total = n_new * R;
    const int n_tiles = (rows_total + 63) / 64;
    if ((int)blockIdx.x >= n_tiles) return;
    const int tile = n_tiles - 1 - blockIdx.x;        // the longest tiles first
    const int row0 = tile * 64;
    const int kv_len = PLM_POSITION(seq_kv_len[b] - 1) + 1;
    const int pos0 = kv_len - n_new;                  // position of the sequence's first new token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)b * max_pages;

    // the tile's query rows: row -> (token = row / R, head = g*R + row % R)
    {
        constexpr int CPR = HD / 8;
        for (int c = threadIdx.x; c < 64 * CPR; c += NT) {
            const int lr = c / CPR, col = c - lr * CPR;
            const int grow = row0 + lr;
            bf16* dst = q_s + lr * LDS + col * 8;
            if (grow < rows_total) {
                const int tok = grow / R, r = grow - tok * R;
                cp_async16(smem_u32(dst), q + ((size_t)(t0 + tok) * H + g * R + r) * HD + col * 8);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
    }
    const int last_row = min(rows_total, row0 + 64) - 1;
    const int pos_min = pos0 + row0 / R, pos_max = pos0 + last_row / R;
    const int first_key = (window > 0 && pos_min - window + 1 > 0) ? pos_min - window + 1 : 0;
    const int page_first = first_key / PLM_PAGE, page_last = pos_max / PLM_PAGE;
    const int n_pages = page_last - page_first + 1;

    auto issue = [&](int i) {                          // page i of this tile's range into stage i % PF_STAGES
        const size_t base = ((size_t)PLM_PAGE_NO(pages[page_first + i]) * G + g) * PLM_PAGE * HD;
        const int valid = kv_len - (page_first + i) * PLM_PAGE;
        load_tile(k_s + (i % PF_STAGES) * TILE_ELEMS, kc + base, valid);
        load_tile(v_s + (i % PF_STAGES) * TILE_ELEMS, vc + base, valid);
    };
    issue(0);
    cp_commit();

    // this thread's two rows
    const int r_lo = row0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    const int pos_lo = r_lo < rows_total ? pos0 + r_lo / R : -1;
    const int pos_hi = r_hi < rows_total ? pos0 + r_hi / R : -1;
    const int lo_lo = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
    const int lo_hi = (window > 0 && pos_hi - window + 1 > 0) ? pos_hi - window + 1 : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int i = 0; i < n_pages; ++i) {
        if (i + 1 < n_pages) issue(i + 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const bf16* kt = k_s + (i % PF_STAGES) * TILE_ELEMS;
        const bf16* vt = v_s + (i % PF_STAGES) * TILE_ELEMS;
        const int key_base = (page_first + i) * PLM_PAGE;
        // a warp whose rows all lie before this page has nothing to do here (causal)
        const int warp_pos_max = pos0 + min(last_row, row0 + warp * 16 + 15) / R;
        if (key_base <= warp_pos_max && row0 + warp * 16 < rows_total) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            qk_tile<8>(s, q_s + warp * 16 * LDS, kt, 0, lane, lane & 15);
            softmax_block<8>(s, o, m, l, scale_log2, key_base, pos_lo, pos_hi, lo_lo, lo_hi, lane);
            pv_tile<8>(o, s, vt, 0, lane);
        }
        __syncthreads();                               // the stage may be overwritten by the next issue
    }
    cp_wait<0>();

    const float inv_lo = l[0] > 0.f ? 1.f / l[0] : 0.f, inv_hi = l[1] > 0.f ? 1.f / l[1] : 0.f;
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
        const int grow = hi ? r_hi : r_lo;
        if (grow >= rows_total) continue;
        const int tok = grow / R, r = grow - tok * R;
        bf16* dst = out + ((size_t)(t0 + tok) * H + g * R + r) * HD + (lane & 3) * 2;
        const float inv = hi ? inv_hi : inv_lo;
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt)
            *reinterpret_cast<uint32_t*>(dst + dt * 8) = pack_bf16(o[dt][2 * hi] * inv, o[dt][2 * hi + 1] * inv);
    }
}

// -------------------------------------------------------------------- decode
constexpr int DC_STAGES = 3;
constexpr size_t DC_TILES_BYTES = (size_t)(2 * DC_STAGES) * TILE_ELEMS * sizeof(bf16);
// Query rows kept in shared memory: all 16 of the MMA's rows, or, for up to 8 query heads per KV head,
// those 8 and one row of zeros that stands for the rest: with head size 64 that lets four CTAs share an SM
// instead of three (57,088 bytes each at most), and a third more bytes are in flight.
constexpr size_t dc_q_bytes(int q_rows) { return (size_t)q_rows * LDS * sizeof(bf16); }
constexpr size_t DC_MERGE_BYTES = (size_t)4 * 16 * (HD + 2) * sizeof(float);
constexpr size_t DC_RESULT_BYTES = (size_t)16 * (HD + 2) * sizeof(float);          // what a CTA shows to its cluster
constexpr size_t DC_AFTER_BYTES = DC_MERGE_BYTES + DC_RESULT_BYTES;
constexpr size_t dc_smem(int q_rows) { return dc_q_bytes(q_rows) + (DC_TILES_BYTES > DC_AFTER_BYTES ? DC_TILES_BYTES : DC_AFTER_BYTES); }
constexpr size_t DC_SMEM = dc_smem(16);
// the TMA form: query rows, then (1024-byte aligned) the ring of unpadded tiles or what follows the loop, then the barriers
constexpr size_t dc_smem_tma(int q_rows) {
    return dc_q_bytes(q_rows) + 1024 +
           ((size_t)2 * DC_STAGES * SW_TILE_BYTES > DC_AFTER_BYTES ? (size_t)2 * DC_STAGES * SW_TILE_BYTES : DC_AFTER_BYTES) + 64;
}
constexpr int DC_MAX_CLUSTER = 8;                                                   // portable cluster size

// grid = (splits, G * row_groups, tokens).  With one split the output is written directly.  With
// CLUSTER the splits of a (token, KV head) are the CTAs of one thread-block cluster: each parks its
// partial result in its own shared memory and the cluster merges them through distributed shared
// memory, in split order.  Without it (more splits than a cluster holds) ws_o [tokens*H, splits, HD]
// and ws_ml [tokens*H, splits, 2] receive the partial results for attn_merge_kernel.
//
// With ROPE the kernel does the rotary encoding and the cache write of the step itself
// (picolm/tensor.c:3216-3304 and picolm/model_core.c:1943-1955 folded in): q is then the output of
// the QKV projection, [tokens, (H + 2G) * HD], the whole head is rotated with half-split pairs by the
// tables rot.cos / rot.sin [positions, HD/2], and the CTAs whose range holds the sequence's last page
// put the step's rotated key and its value into their copy of that page; those of the first row
// group also write them to the cache.  No other kernel of the step then writes this cache, so every
// page may be requested before the kernel in front has finished.
struct Rotary {
    const float* cos;
    const float* sin;
    bf16* kc_w;          // the cache, writable
    bf16* vc_w;
};

// x[j..j+8) and x[HD/2+j..HD/2+j+8) of one head, rotated by the angles of `pos` (fp32, rounded once)
__device__ __forceinline__ void rotate16(uint4& lo, uint4& hi, const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t, int pos, int j) {
    const float* cp = cos_t + (size_t)pos * (HD / 2) + j;
    const float* sp = sin_t + (size_t)pos * (HD / 2) + j;
    __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float a0 = __low2float(l2[k]), a1 = __high2float(l2[k]);
        const float b0 = __low2float(h2[k]), b1 = __high2float(h2[k]);
        const float c0 = cp[2 * k], c1 = cp[2 * k + 1], s0 = sp[2 * k], s1 = sp[2 * k + 1];
        l2[k] = __floats2bfloat162_rn(rope_first(a0, b0, c0, s0), rope_first(a1, b1, c1, s1));
        h2[k] = __floats2bfloat162_rn(rope_second(a0, b0, c0, s0), rope_second(a1, b1, c1, s1));
    }
}

struct PageMaps {               // the TMA form: the caches as [pages * G * 64 rows, HD], boxes of 64 x 64
    CUtensorMap k, v;
};

template <bool CLUSTER, bool ROPE, bool TMA>
__global__ void __launch_bounds__(NT)
attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                   bf16* __restrict__ out, float* __restrict__ ws_o, float* __restrict__ ws_ml,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                   int max_pages, int H, int G, float scale_log2, int window, int row_groups, const Rotary rot,
                   int q_rows, const __grid_constant__ PageMaps maps, int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const size_t q_bytes = (size_t)q_rows * LDS * sizeof(bf16);          // q_rows: 16, or 9 (8 heads and a row of zeros)
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);
    // after the query rows: the ring of tiles (padded for cp.async; 1024-byte aligned and unpadded for TMA)
    const uint32_t ring = TMA ? ((smem_u32(smem_raw) + (uint32_t)q_bytes + 1023u) & ~1023u) : smem_u32(smem_raw) + (uint32_t)q_bytes;
    uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    bf16* k_s = reinterpret_cast<bf16*>(ring_ptr);
    bf16* v_s = k_s + DC_STAGES * TILE_ELEMS;
    float* merge = reinterpret_cast<float*>(ring_ptr);                   // reused after the last tile
    float* result = reinterpret_cast<float*>(ring_ptr + DC_MERGE_BYTES);
    constexpr size_t RING_BYTES = (size_t)2 * DC_STAGES * SW_TILE_BYTES > DC_AFTER_BYTES ? (size_t)2 * DC_STAGES * SW_TILE_BYTES : DC_AFTER_BYTES;
    const uint32_t full0 = ring + (uint32_t)RING_BYTES;                   // TMA: one barrier a stage
    if (TMA && threadIdx.x == 0) {
        for (int s = 0; s < DC_STAGES; ++s) plm_tc::mbar_init(full0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (TMA) __syncthreads();
    pdl_launch_dependents();
    // What describes the step (positions, page tables) was written before the step began, and pages
    // before a sequence's last one hold keys of earlier steps: all of that may be read before the
    // kernel in front of this one (which writes this step's key and the queries) has finished.
    const int n_splits = gridDim.x, split = blockIdx.x;
    const int g = blockIdx.y / row_groups, rg = blockIdx.y - g * row_groups;
    const int t = blockIdx.z;
    const int R = H / G;
    const int h0 = g * R + rg * 16;                     // first head of this row group
    const int n_rows = min(16, R - rg * 16);
    const int pos = PLM_POSITION(tok_pos[t]);
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int page_first = lo / PLM_PAGE, page_last = pos / PLM_PAGE;
    const int total_pages = page_last - page_first + 1;
    const int per = (total_pages + n_splits - 1) / n_splits;
    const int p_begin = page_first + split * per;
    const int p_end = min(page_last + 1, p_begin + per);
    const int n_pages = p_end - p_begin;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages;

    auto issue = [&](int i) {
        if constexpr (TMA) {
            if (threadIdx.x == 0) {                     // a page's keys and values: HD / 64 boxes each, one barrier
                const int st = i % DC_STAGES;
                const int row0 = (PLM_PAGE_NO(pages[p_begin + i]) * G + g) * PLM_PAGE;
                const uint32_t kd = ring + (uint32_t)(2 * st) * SW_TILE_BYTES, vd = kd + SW_TILE_BYTES;
                plm_tc::mbar_expect_tx(full0 + 8 * st, 2 * SW_TILE_BYTES);
#pragma unroll
                for (int sub = 0; sub < HD / 64; ++sub) {
                    plm_tc::tma_load_2d(kd + sub * 8192, &maps.k, full0 + 8 * st, sub * 64, row0);
                    plm_tc::tma_load_2d(vd + sub * 8192, &maps.v, full0 + 8 * st, sub * 64, row0);
                }
            }
        } else {
            const size_t base = ((size_t)PLM_PAGE_NO(pages[p_begin + i]) * G + g) * PLM_PAGE * HD;
            const int valid = pos + 1 - (p_begin + i) * PLM_PAGE;
            load_tile(k_s + (i % DC_STAGES) * TILE_ELEMS, kc + base, valid);
            load_tile(v_s + (i % DC_STAGES) * TILE_ELEMS, vc + base, valid);
        }
    };
    const int n_first = min(n_pages, DC_STAGES - 1);                    // pages asked for before the loop
    const bool early = ROPE || n_first <= 0 || p_begin + n_first - 1 < page_last;  // none of them is written in this step
    if (!early) pdl_wait();
#pragma unroll
    for (int i = 0; i < DC_STAGES - 1; ++i) {
        if (i < n_pages) issue(i);
        if (!TMA) cp_commit();
    }
    if (early) pdl_wait();
    if (!CLUSTER && n_pages <= 0) {                     // an empty split: weight zero in the merge
        for (int r = threadIdx.x; r < n_rows; r += NT) {
            float* ml = ws_ml + (((size_t)t * H + h0 + r) * n_splits + split) * 2;
            ml[0] = -INFINITY; ml[1] = 0.f;
        }
        return;
    }
    if (n_pages > 0 && !ROPE) {                         // (in a cluster an empty split still meets the others)
        constexpr int CPR = HD / 8;                     // the queries: plain loads, visible after the loop's first barrier
        for (int c = threadIdx.x; c < q_rows * CPR; c += NT) {
            const int r = c / CPR, col = c - r * CPR;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n_rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * H + h0 + r) * HD + col * 8);
            *reinterpret_cast<uint4*>(q_s + r * LDS + col * 8) = v;
        }
    }
    const bf16* qkv_row = q + (size_t)t * (H + 2 * G) * HD;              // ROPE: this token's projections
    if (n_pages > 0 && ROPE) {
        constexpr int GRP = HD / 16;                    // groups of 8 pairs per head
        for (int c = threadIdx.x; c < q_rows * GRP; c += NT) {
            const int r = c / GRP, j = (c - r * GRP) * 8;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
            if (r < n_rows) {
                lo = *reinterpret_cast<const uint4*>(qkv_row + (size_t)(h0 + r) * HD + j);
                hi = *reinterpret_cast<const uint4*>(qkv_row + (size_t)(h0 + r) * HD + HD / 2 + j);
                rotate16(lo, hi, rot.cos, rot.sin, pos, j);
            }
            *reinterpret_cast<uint4*>(q_s + r * LDS + j) = lo;
            *reinterpret_cast<uint4*>(q_s + r * LDS + HD / 2 + j) = hi;
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int i = 0; i < n_pages; ++i) {
        if (i + DC_STAGES - 1 < n_pages) issue(i + DC_STAGES - 1);
        const uint32_t kt_sw = ring + (uint32_t)(2 * (i % DC_STAGES)) * SW_TILE_BYTES, vt_sw = kt_sw + SW_TILE_BYTES;
        if constexpr (TMA) {
            // (the stage that was just asked for again was released by the barrier that ended the iteration before)
            plm_tc::mbar_wait(full0 + 8 * (i % DC_STAGES), (uint32_t)((i / DC_STAGES) & 1), status, 5);
            if (i == 0) __syncthreads();                // the query rows, written with plain stores above
            if (p_begin + i == page_last) {
                // Places of the page that hold no key yet may hold whatever an earlier owner of the page left:
                // zeros instead, so that nothing of it reaches a sum (a masked score times a stale value).
                const int first_free = pos + (ROPE ? 0 : 1) - page_last * PLM_PAGE;     // ROPE: this step's row is written below
                for (int c = threadIdx.x; c < (PLM_PAGE - first_free) * (HD / 8); c += NT) {
                    const int r = first_free + c / (HD / 8), ch = c % (HD / 8);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(kt_sw + sw_off(r, ch)), "r"(0u) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vt_sw + sw_off(r, ch)), "r"(0u) : "memory");
                }
                __syncthreads();
            }
        } else {
            cp_commit();
            cp_wait<DC_STAGES - 1>();
            __syncthreads();
        }
        const bf16* kt = k_s + (i % DC_STAGES) * TILE_ELEMS;
        const bf16* vt = v_s + (i % DC_STAGES) * TILE_ELEMS;
        if (ROPE && p_begin + i == page_last) {
            // the step's own key (rotated) and value: into this CTA's copy of the page, and from the
            // first row group into the cache as well
            constexpr int GRP = HD / 16;
            const int in_page = pos - page_last * PLM_PAGE;
            bf16* k_row = k_s + (i % DC_STAGES) * TILE_ELEMS + in_page * LDS;
            bf16* v_row = v_s + (i % DC_STAGES) * TILE_ELEMS + in_page * LDS;
            const int own_page = PLM_PAGE_NO(pages[page_last]);
            const size_t cache_row = (((size_t)own_page * G + g) * PLM_PAGE + in_page) * HD;
            const bool to_cache = rg == 0 && own_page > 0;       // page 0 is the null page of padding rows
            if (threadIdx.x < GRP) {
                const int j = threadIdx.x * 8;
                uint4 lo = *reinterpret_cast<const uint4*>(qkv_row + (size_t)(H + g) * HD + j);
                uint4 hi = *reinterpret_cast<const uint4*>(qkv_row + (size_t)(H + g) * HD + HD / 2 + j);
                rotate16(lo, hi, rot.cos, rot.sin, pos, j);
                if constexpr (TMA) {
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(kt_sw + sw_off(in_page, j / 8)),
                                 "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(kt_sw + sw_off(in_page, (HD / 2 + j) / 8)),
                                 "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
                } else {
                    *reinterpret_cast<uint4*>(k_row + j) = lo;
                    *reinterpret_cast<uint4*>(k_row + HD / 2 + j) = hi;
                }
                if (to_cache) {
                    *reinterpret_cast<uint4*>(rot.kc_w + cache_row + j) = lo;
                    *reinterpret_cast<uint4*>(rot.kc_w + cache_row + HD / 2 + j) = hi;
                }
            } else if (threadIdx.x >= 32 && threadIdx.x < 32 + HD / 8) {
                const int j = (threadIdx.x - 32) * 8;
                const uint4 v = *reinterpret_cast<const uint4*>(qkv_row + (size_t)(H + G + g) * HD + j);
                if constexpr (TMA)
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(vt_sw + sw_off(in_page, j / 8)),
                                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                else
                    *reinterpret_cast<uint4*>(v_row + j) = v;
                if (to_cache) *reinterpret_cast<uint4*>(rot.vc_w + cache_row + j) = v;
            }
            __syncthreads();
        }
        const int key_base = (p_begin + i) * PLM_PAGE + warp * 16;       // this warp's 16 keys of the page
        if (key_base <= pos) {
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            if constexpr (TMA) {
                qk_tile_sw<2>(s, q_s, kt_sw, warp * 16, lane, min(lane & 15, q_rows - 1));
                softmax_block<2>(s, o, m, l, scale_log2, key_base, pos, pos, lo, lo, lane);
                pv_tile_sw<2>(o, s, vt_sw, warp * 16, lane);
            } else {
                qk_tile<2>(s, q_s, kt, warp * 16, lane, min(lane & 15, q_rows - 1));
                softmax_block<2>(s, o, m, l, scale_log2, key_base, pos, pos, lo, lo, lane);
                pv_tile<2>(o, s, vt, warp * 16, lane);
            }
        }
        __syncthreads();
    }
    if (!TMA) cp_wait<0>();
    __syncthreads();

    // merge the four warps' partial results: merge[w][row][0..HD) = acc, [HD] = m, [HD+1] = l
    // (a split without pages leaves m = -inf and l = 0 here: weight zero below)
    {
        float* mine = merge + (size_t)warp * 16 * (HD + 2);
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            const int r = (lane >> 2) + hi * 8;
#pragma unroll
            for (int dt = 0; dt < HD / 8; ++dt) {
                mine[r * (HD + 2) + dt * 8 + (lane & 3) * 2] = o[dt][2 * hi];
                mine[r * (HD + 2) + dt * 8 + (lane & 3) * 2 + 1] = o[dt][2 * hi + 1];
            }
            if ((lane & 3) == 0) {
                mine[r * (HD + 2) + HD] = m[hi];
                mine[r * (HD + 2) + HD + 1] = l[hi];
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_rows * HD; idx += NT) {
        const int r = idx / HD, d = idx - r * HD;
        float mw[4], mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            mw[w] = merge[((size_t)w * 16 + r) * (HD + 2) + HD];
            mm = fmaxf(mm, mw[w]);
        }
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - mm);
            acc += wgt * merge[((size_t)w * 16 + r) * (HD + 2) + d];
            ll += wgt * merge[((size_t)w * 16 + r) * (HD + 2) + HD + 1];
        }
        const size_t row = (size_t)t * H + h0 + r;
        if (CLUSTER) {
            result[r * (HD + 2) + d] = acc;
            if (d == 0) {
                result[r * (HD + 2) + HD] = mm;
                result[r * (HD + 2) + HD + 1] = ll;
            }
        } else if (n_splits == 1) {
            out[row * HD + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        } else {
            ws_o[(row * n_splits + split) * HD + d] = acc;
            if (d == 0) {
                ws_ml[(row * n_splits + split) * 2] = mm;
                ws_ml[(row * n_splits + split) * 2 + 1] = ll;
            }
        }
    }
    if (CLUSTER) {
        // out[row, :] = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp2(m_s - max m), splits in order;
        // the outputs are dealt out over the cluster's CTAs
        cluster_sync_all();
        const uint32_t rank = cluster_rank();           // == split: the cluster spans grid x
        for (int idx = (int)rank * NT + threadIdx.x; idx < n_rows * HD; idx += n_splits * NT) {
            const int r = idx / HD, d = idx - r * HD;
            float ms[DC_MAX_CLUSTER], ls[DC_MAX_CLUSTER], as[DC_MAX_CLUSTER];
#pragma unroll
            for (int sp = 0; sp < DC_MAX_CLUSTER; ++sp) {
                if (sp < n_splits) {
                    const uint32_t base = cluster_map(result + r * (HD + 2), (uint32_t)sp);
                    ms[sp] = cluster_ld_f32(base + HD * 4);
                    ls[sp] = cluster_ld_f32(base + (HD + 1) * 4);
                    as[sp] = cluster_ld_f32(base + d * 4);
                } else {
                    ms[sp] = -INFINITY; ls[sp] = 0.f; as[sp] = 0.f;
                }
            }
            float mm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < DC_MAX_CLUSTER; ++sp) mm = fmaxf(mm, ms[sp]);
            float acc = 0.f, ll = 0.f;
#pragma unroll
            for (int sp = 0; sp < DC_MAX_CLUSTER; ++sp) {
                if (ms[sp] == -INFINITY) continue;
                const float wgt = exp2f(ms[sp] - mm);
                acc += wgt * as[sp];
                ll += wgt * ls[sp];
            }
            out[((size_t)t * H + h0 + r) * HD + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        }
        cluster_sync_all();                             // nobody reads this CTA's shared memory any more
    }
}

// out[row, :] = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp2(m_s - max m): one block per (token, head).
// 256 threads: the ranges' maxima and weights are found by all threads side by side; then MERGE_GROUPS groups of
// MERGE_LANES threads (one per component) each add up a stretch of the ranges, with the loads of eight ranges in
// flight, and the stretches' sums are added in their order: always the same order for a number of ranges.
constexpr int MERGE_THREADS = 256;
constexpr int MERGE_MAX_SPLITS = 8192;                   // the weights of all ranges lie in shared memory
constexpr int MERGE_LANES = HD <= 64 ? 64 : HD <= 128 ? 128 : 256;
constexpr int MERGE_GROUPS = MERGE_THREADS / MERGE_LANES;
__global__ void __launch_bounds__(MERGE_THREADS)
attn_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, bf16* __restrict__ out, int n_splits) {
    extern __shared__ float merge_w[];                  // [n_splits] weights, then [MERGE_GROUPS][MERGE_LANES] sums
    __shared__ float red[MERGE_THREADS / 32];
    __shared__ float s_max, s_l;
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* ml = ws_ml + row * n_splits * 2;
    float m = -INFINITY;
    for (int s = tid; s < n_splits; s += MERGE_THREADS) m = fmaxf(m, ml[2 * s]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float mm = red[0];
        for (int w = 1; w < MERGE_THREADS / 32; ++w) mm = fmaxf(mm, red[w]);
        s_max = mm;
    }
    __syncthreads();
    const float mm = s_max;
    for (int s = tid; s < n_splits; s += MERGE_THREADS) {
        const float ms = ml[2 * s];
        merge_w[s] = ms == -INFINITY ? 0.f : exp2f(ms - mm);
    }
    __syncthreads();
    if (warp == 0) {                                    // the sum of the weighted row sums, ranges in order
        float ll = 0.f;
        if (lane == 0)
            for (int s = 0; s < n_splits; ++s)
                if (merge_w[s] != 0.f) ll += merge_w[s] * ml[2 * s + 1];
        if (lane == 0) s_l = ll;
    }
    float* sums = merge_w + n_splits;
    const int g = tid / MERGE_LANES, d = tid % MERGE_LANES;
    const int per = (n_splits + MERGE_GROUPS - 1) / MERGE_GROUPS;
    const int s_begin = g * per, s_end = min(n_splits, s_begin + per);
    float acc = 0.f;
    if (d < HD) {
        const float* o = ws_o + row * n_splits * HD + d;
        int s = s_begin;
        for (; s + 8 <= s_end; s += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = o[(size_t)(s + i) * HD];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (merge_w[s + i] != 0.f) acc += merge_w[s + i] * v[i];   // an empty range left nothing to read
        }
        for (; s < s_end; ++s)
            if (merge_w[s] != 0.f) acc += merge_w[s] * o[(size_t)s * HD];
    }
    sums[g * MERGE_LANES + d] = acc;
    __syncthreads();
    if (g == 0 && d < HD) {
        float total = sums[d];
        for (int k = 1; k < MERGE_GROUPS; ++k) total += sums[k * MERGE_LANES + d];
        const float ll = s_l;
        out[row * HD + d] = __float2bfloat16_rn(ll > 0.f ? total / ll : 0.f);
    }
}

// 9 query rows (8 heads and a row of zeros) make room for a fourth CTA on an SM.  That pays where the grid
// is several waves long (large batches: a third more bytes in flight); a grid of one wave runs better with
// three, which leave room for the CTAs of the kernel behind it to ask for their weights meanwhile.
int decode_q_rows(int heads_per_kv_head, long ctas) { return heads_per_kv_head <= 8 && ctas > 3 * PLM_SM_COUNT ? 9 : 16; }

// The caches as TMA sees them: [n_pages * G * 64 rows, HD] bf16, boxes of 64 rows x 64 columns, 128-byte swizzle.
int page_maps(PageMaps* maps, const void* kc, const void* vc, int n_pages, int G) {
    const long rows = (long)n_pages * G * PLM_PAGE;
    int rc = plm_tc::make_map(&maps->k, kc, rows, HD, HD, 64);
    if (rc == PLM_OK) rc = plm_tc::make_map(&maps->v, vc, rows, HD, HD, 64);
    return rc;
}

template <typename K>
int set_smem(K kern, size_t bytes) {
    if (bytes <= 48 * 1024) return PLM_OK;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return e == cudaSuccess ? PLM_OK : (int)e;
}

}  // namespace

extern "C" int plm_attn_head_dim() { return HD; }

// Prefill: q [T, H, HD], out [T, H*HD]; the step's sequences are described by seq_start [B+1]
// (offsets of each sequence's new tokens) and seq_kv_len [B] (length after the step);
// max_new is the largest number of new tokens of a sequence.
extern "C" int plm_attn_prefill(const void* q, const void* kc, const void* vc, void* out, const int* seq_start,
                                const int* seq_kv_len, const int* block_table, int max_pages, int n_seqs, int max_new,
                                int H, int G, float scale, int window, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || H % G || n_seqs > 65535 || G > 65535) return PLM_ERR_SHAPE;
    static bool configured = false;
    if (!configured) {
        int rc = set_smem(attn_prefill_kernel, PF_SMEM);
        if (rc != PLM_OK) return rc;
        configured = true;
    }
    const int R = H / G;
    dim3 grid(((size_t)max_new * R + 63) / 64, G, n_seqs);
    return plm_status_of(launch_pdl(attn_prefill_kernel, grid, dim3(NT), PF_SMEM, stream, (const bf16*)q, (const bf16*)kc,
                                    (const bf16*)vc, (bf16*)out, seq_start, seq_kv_len, block_table, max_pages, H, G,
                                    scale * LOG2E, window));
}

// Floats of workspace that plm_attn_decode needs for (tokens, H, splits): acc then (m, l).
extern "C" long plm_attn_decode_workspace(int n_tokens, int H, int n_splits) {
    return n_splits > 1 ? (long)n_tokens * H * n_splits * (HD + 2) : 0;
}

// Decode: one query token per row of q [T, H, HD], at position tok_pos[t] of sequence tok_seq[t].
// With a workspace the ranges' partial results pass through it and a second kernel merges them;
// without one (at most 8 ranges) the ranges are the CTAs of a cluster and merge in shared memory.
// `n_pages`: pages of the cache (kc and vc are [n_pages, G, 64, HD]); `status`: the device word that a wait
// which runs out writes to (head sizes that are multiples of 64 ask for pages by TMA and wait on barriers).
extern "C" int plm_attn_decode(const void* q, const void* kc, const void* vc, void* out, float* workspace,
                               const int* tok_pos, const int* tok_seq, const int* block_table, int max_pages,
                               int n_tokens, int H, int G, float scale, int window, int n_splits, int n_pages,
                               int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || H % G || n_splits < 1 || n_tokens > 65535) return PLM_ERR_SHAPE;
    constexpr bool TMA = HAS_TMA;
    static bool configured = false;
    if (!configured) {
        int rc = set_smem(attn_decode_kernel<false, false, TMA>, TMA ? dc_smem_tma(16) : DC_SMEM);
        if (rc == PLM_OK) rc = set_smem(attn_decode_kernel<true, false, TMA>, TMA ? dc_smem_tma(16) : DC_SMEM);
        if (rc != PLM_OK) return rc;
        configured = true;
    }
    PageMaps maps = {};
    if (TMA) {
        if (n_pages <= 0 || !status) return PLM_ERR_SHAPE;
        int rc = page_maps(&maps, kc, vc, n_pages, G);
        if (rc != PLM_OK) return rc;
    }
    const int R = H / G, row_groups = (R + 15) / 16;
    if (G * row_groups > 65535) return PLM_ERR_SHAPE;
    const int q_rows = decode_q_rows(R, (long)n_splits * G * row_groups * n_tokens);
    const size_t smem = TMA ? dc_smem_tma(q_rows) : dc_smem(q_rows);
    dim3 grid(n_splits, G * row_groups, n_tokens);
    if (n_splits > MERGE_MAX_SPLITS) return PLM_ERR_SHAPE;
    if (n_splits > 1 && !workspace) {                       // the splits merge inside their cluster
        if (n_splits > DC_MAX_CLUSTER) return PLM_ERR_SHAPE;
        return plm_status_of(launch_pdl_cluster(attn_decode_kernel<true, false, TMA>, grid, dim3(NT), dim3(n_splits, 1, 1), smem,
                                                stream, (const bf16*)q, (const bf16*)kc, (const bf16*)vc, (bf16*)out,
                                                (float*)nullptr, (float*)nullptr, tok_pos, tok_seq, block_table,
                                                max_pages, H, G, scale * LOG2E, window, row_groups, Rotary{}, q_rows, maps, status));
    }
    float* ws_o = workspace;
    float* ws_ml = workspace ? workspace + (size_t)n_tokens * H * n_splits * HD : nullptr;
    int rc = plm_status_of(launch_pdl(attn_decode_kernel<false, false, TMA>, grid, dim3(NT), smem, stream, (const bf16*)q,
                                      (const bf16*)kc, (const bf16*)vc, (bf16*)out, ws_o, ws_ml, tok_pos, tok_seq,
                                      block_table, max_pages, H, G, scale * LOG2E, window, row_groups, Rotary{}, q_rows, maps, status));
    if (rc != PLM_OK || n_splits == 1) return rc;
    return plm_status_of(launch_pdl(attn_merge_kernel, dim3(n_tokens * H), dim3(MERGE_THREADS),
                                    (size_t)(n_splits + MERGE_THREADS) * sizeof(float), stream,
                                    (const float*)ws_o, (const float*)ws_ml, (bf16*)out, n_splits));
}

// Decode with the rotary encoding and the cache write folded in (see struct Rotary): qkv [T, (H + 2G) * HD]
// is the QKV projection's output, cos_t / sin_t [positions, HD/2] fp32; the step's keys and values are
// written to kc / vc at tok_pos.  Otherwise as plm_attn_decode.
extern "C" int plm_attn_decode_rope(const void* qkv, void* kc, void* vc, void* out, float* workspace,
                                    const float* cos_t, const float* sin_t, const int* tok_pos, const int* tok_seq,
                                    const int* block_table, int max_pages, int n_tokens, int H, int G, float scale,
                                    int window, int n_splits, int n_pages, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || H % G || n_splits < 1 || n_tokens > 65535 || !cos_t || !sin_t) return PLM_ERR_SHAPE;
    constexpr bool TMA = HAS_TMA;
    static bool configured = false;
    if (!configured) {
        int rc = set_smem(attn_decode_kernel<false, true, TMA>, TMA ? dc_smem_tma(16) : DC_SMEM);
        if (rc == PLM_OK) rc = set_smem(attn_decode_kernel<true, true, TMA>, TMA ? dc_smem_tma(16) : DC_SMEM);
        if (rc != PLM_OK) return rc;
        configured = true;
    }
    PageMaps maps = {};
    if (TMA) {
        if (n_pages <= 0 || !status) return PLM_ERR_SHAPE;
        int rc = page_maps(&maps, kc, vc, n_pages, G);
        if (rc != PLM_OK) return rc;
    }
    const int R = H / G, row_groups = (R + 15) / 16;
    if (G * row_groups > 65535) return PLM_ERR_SHAPE;
    const Rotary rot = {cos_t, sin_t, (bf16*)kc, (bf16*)vc};
    const int q_rows = decode_q_rows(R, (long)n_splits * G * row_groups * n_tokens);
    const size_t smem = TMA ? dc_smem_tma(q_rows) : dc_smem(q_rows);
    dim3 grid(n_splits, G * row_groups, n_tokens);
    if (n_splits > MERGE_MAX_SPLITS) return PLM_ERR_SHAPE;
    if (n_splits > 1 && !workspace) {
        if (n_splits > DC_MAX_CLUSTER) return PLM_ERR_SHAPE;
        return plm_status_of(launch_pdl_cluster(attn_decode_kernel<true, true, TMA>, grid, dim3(NT), dim3(n_splits, 1, 1), smem,
                                                stream, (const bf16*)qkv, (const bf16*)kc, (const bf16*)vc, (bf16*)out,
                                                (float*)nullptr, (float*)nullptr, tok_pos, tok_seq, block_table,
                                                max_pages, H, G, scale * LOG2E, window, row_groups, rot, q_rows, maps, status));
    }
    float* ws_o = workspace;
    float* ws_ml = workspace ? workspace + (size_t)n_tokens * H * n_splits * HD : nullptr;
    int rc = plm_status_of(launch_pdl(attn_decode_kernel<false, true, TMA>, grid, dim3(NT), smem, stream, (const bf16*)qkv,
                                      (const bf16*)kc, (const bf16*)vc, (bf16*)out, ws_o, ws_ml, tok_pos, tok_seq,
                                      block_table, max_pages, H, G, scale * LOG2E, window, row_groups, rot, q_rows, maps, status));
    if (rc != PLM_OK || n_splits == 1) return rc;
    return plm_status_of(launch_pdl(attn_merge_kernel, dim3(n_tokens * H), dim3(MERGE_THREADS),
                                    (size_t)(n_splits + MERGE_THREADS) * sizeof(float), stream,
                                    (const float*)ws_o, (const float*)ws_ml, (bf16*)out, n_splits));
}
