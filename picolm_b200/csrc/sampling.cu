// Token selection from fp32 logits on the device: greedy argmax and the
// reference's sampling chain softmax -> top-k -> top-p -> min-p -> p^(1/T) -> draw
// (picolm/sampler.c:48-125).  One thread-block cluster of eight CTAs per sequence:
// each CTA keeps an eighth of the row's probabilities in its shared memory, and
// the CTAs exchange their partial results (maxima, sums, histograms) through
// distributed shared memory.
//
// The reference sorts the probabilities and cuts the sorted list; a cut of a
// sorted list is the set {p >= threshold}, so the kept set is found here without
// a sort, by a radix select on the probabilities' bit patterns (8 bits a pass):
// the k-th largest value for top-k, and the value at which the mass of everything
// at or above it reaches top-p.  Values that tie with the value at the cut are all
// kept.  The draw walks the kept tokens in index order (the reference walks them
// in sorted order): the same distribution, another token for a given random
// number.  Random numbers are the reference's xorshift64 stream
// (picolm/sampler.c:10-21), one state per sequence, advanced in place.
// Everything is summed in a fixed order (masses as 2^-40 fixed-point integers), so
// the same inputs give the same token.
#include "common.cuh"
#include <limits.h>

namespace {

constexpr int NT = 256;
constexpr int CS = 8;                         // CTAs per cluster (one cluster per row)
constexpr int MAX_CHUNK = 40 * 1024;          // floats of a row's eighth that fit a CTA's shared memory
constexpr float FIX = 1099511627776.0f;       // 2^40: probabilities as fixed-point integers
constexpr int BINS = 1024;                    // a radix digit has 10 bits
constexpr int SLICE = BINS / CS;              // bins that one CTA merges over the cluster

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ldc_f32(uint32_t a) { float v; asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ int ldc_s32(uint32_t a) { int v; asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ unsigned long long ldc_u64(uint32_t a) { unsigned long long v; asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ uint4 ldc_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
    return v;
}

// What a CTA shows to the others of its cluster.
struct Shared {
    float max_v; int max_i;                   // local maximum and its first index
    float sum;                                // local sum (of exp, later of the kept weights)
    int cand;                                 // local candidate of the draw
};

__device__ __forceinline__ float block_sum_f(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < NT / 32 ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// What the radix select of a CTA shows to the others.
struct Radix {
    // radix histogram of the current pass: a count and the mass as three limbs of 14 bits per bin
    // (shared memory adds 32-bit words natively; 40,960 values of 14 bits stay below 2^32)
    alignas(16) unsigned hist[BINS * 4];
    long long slice_cnt;                      // totals of the bins this CTA merges
    unsigned long long slice_mass;
    int res_k_digit, res_p_digit;             // what the owner of the crossing found
    long long res_k_before;
    unsigned long long res_p_before;
};

// Run by one warp over a slice of SLICE bins: the highest bin at which the running total from the top
// (starting at `above`) reaches `left`, and the total before that bin.  The caller knows there is one.
__device__ void slice_crossing(const unsigned long long* bins, unsigned long long above, unsigned long long left, int& digit,
                               unsigned long long& before) {
    constexpr int PER = SLICE / 32;
    const int lane = threadIdx.x & 31;
    unsigned long long v[PER], mine = 0ull;
#pragma unroll
    for (int j = 0; j < PER; ++j) { v[j] = bins[lane * PER + j]; mine += v[j]; }
    unsigned long long run = above;                      // plus everything in higher lanes
    for (int l = 31; l > 0; --l) {
        const unsigned long long o = __shfl_sync(0xffffffffu, mine, l);
        if (l > lane) run += o;
    }
    int d = -1;
    unsigned long long b = 0ull;
#pragma unroll
    for (int j = PER - 1; j >= 0; --j) {
        if (d < 0 && run < left && run + v[j] >= left) { d = lane * PER + j; b = run; }
        run += v[j];
    }
    const unsigned found = __ballot_sync(0xffffffffu, d >= 0);
    const int src = found ? 31 - __clz(found) : 0;       // the highest lane that has one
    digit = __shfl_sync(0xffffffffu, d, src);
    before = __shfl_sync(0xffffffffu, b, src);
    if (!found) { digit = 0; before = 0ull; }
}

// The row's maximum and the first index that has it, over the whole cluster (strict > scan from
// index 0, picolm/sampler.c:50-56).  Every CTA returns the same pair.
__device__ void cluster_argmax(const float* __restrict__ row, int lo, int hi, Shared* sh, float* redf, int* redi,
                               float& best_v, int& best_i) {
    float bv = -INFINITY;
    int bi = INT_MAX;
    for (int i = lo + threadIdx.x; i < hi; i += NT) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }                  // ascending i per thread: the first index wins ties
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { redf[warp] = bv; redi[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < NT / 32; ++w)
            if (redf[w] > bv || (redf[w] == bv && redi[w] < bi)) { bv = redf[w]; bi = redi[w]; }
        sh->max_v = bv;
        sh->max_i = bi;
    }
    cluster_sync_all();
    best_v = -INFINITY;
    best_i = INT_MAX;
    float vs[CS];
    int is[CS];
#pragma unroll
    for (uint32_t r = 0; r < CS; ++r) {
        vs[r] = ldc_f32(map_to_rank(smem_addr(&sh->max_v), r));
        is[r] = ldc_s32(map_to_rank(smem_addr(&sh->max_i), r));
    }
#pragma unroll
    for (uint32_t r = 0; r < CS; ++r)
        if (vs[r] > best_v || (vs[r] == best_v && is[r] < best_i)) { best_v = vs[r]; best_i = is[r]; }
    if (best_i == INT_MAX) best_i = 0;                   // a row of NaN or -inf: the reference answers 0
}

__global__ void __launch_bounds__(NT)
argmax_kernel(const float* __restrict__ logits, long ld, int V, int chunk, int* __restrict__ out) {
    __shared__ Shared sh;
    __shared__ float redf[33];
    __shared__ int redi[33];
    pdl_launch_dependents();
    pdl_wait();
    const int row_id = blockIdx.x / CS;
    const uint32_t rank = cluster_rank();
    const float* row = logits + (size_t)row_id * ld;
    const int lo = min(V, (int)rank * chunk), hi = min(V, lo + chunk);
    float bv;
    int bi;
    cluster_argmax(row, lo, hi, &sh, redf, redi, bv, bi);
    if (rank == 0 && threadIdx.x == 0) out[row_id] = bi;
    cluster_sync_all();                                  // nobody reads this CTA's shared memory any more
}

__global__ void __launch_bounds__(NT, 2)
sample_kernel(const float* __restrict__ logits, long ld, int V, int chunk, float temperature, int top_k, float top_p,
              float min_p, unsigned long long* __restrict__ rng, int* __restrict__ out) {
    extern __shared__ float prob[];                      // this CTA's eighth of the row's probabilities
    __shared__ Shared sh;
    __shared__ float redf[33];
    __shared__ int redi[33];
    __shared__ Radix rx;
    __shared__ unsigned long long s_cbin[SLICE];
    __shared__ unsigned long long s_mbin[SLICE];
    pdl_launch_dependents();
    pdl_wait();
    const int row_id = blockIdx.x / CS;
    const uint32_t rank = cluster_rank();
    const float* row = logits + (size_t)row_id * ld;
    const int lo = min(V, (int)rank * chunk), hi = min(V, lo + chunk), n = hi - lo;
    const int tid = threadIdx.x;

    // ---- softmax of the raw logits (picolm/tensor.c:3066-3076): max, exp, sum, scale
    float mx;
    int best;
    cluster_argmax(row, lo, hi, &sh, redf, redi, mx, best);
    float z = 0.f;
    for (int i = tid; i < n; i += NT) {
        const float e = expf(row[lo + i] - mx);
        prob[i] = e;
        z += e;
    }
    z = block_sum_f(z, redf);
    if (tid == 0) sh.sum = z;
    cluster_sync_all();
    float zs[CS];
#pragma unroll
    for (uint32_t r = 0; r < CS; ++r) zs[r] = ldc_f32(map_to_rank(smem_addr(&sh.sum), r));
    float total = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < CS; ++r) total += zs[r];                                          // rank order
    const float inv = 1.0f / total;
    for (int i = tid; i < n; i += NT) prob[i] *= inv;
    __syncthreads();
    cluster_sync_all();                                  // everyone has read the sums; sh.sum is reused below

    // ---- thresholds by radix select on the bit patterns (positive floats order like their bits).
    // A probability is at most 1, so its two highest bits are 0: three digits of 10 bits cover it, and
    // the first one (the exponent and two bits of the mantissa) already spreads a row over a hundred bins.
    const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.0f;
    unsigned thr_k = 0u, thr_p = 0u;
    long long k_left = top_k;
    unsigned long long p_left = (unsigned long long)((double)top_p * (double)FIX);
    bool k_done = !use_k, p_done = !use_p;
    for (int shift = 20; shift >= 0 && !(k_done && p_done); shift -= 10) {
        for (int b = tid; b < BINS * 4; b += NT) rx.hist[b] = 0u;
        __syncthreads();
        const unsigned hi_mask = 0xffffffffu << (shift + 10);
        for (int i = tid; i < n; i += NT) {
            const float p = prob[i];
            const unsigned bits = __float_as_uint(p);
            const unsigned d = (bits >> shift) & (BINS - 1);
            if (!k_done && (bits & hi_mask) == (thr_k & hi_mask)) atomicAdd(&rx.hist[d * 4], 1u);
            if (!p_done && (bits & hi_mask) == (thr_p & hi_mask)) {
                const unsigned long long m = __float2ull_rn(p * FIX);               // at most 2^40
                atomicAdd(&rx.hist[d * 4 + 1], (unsigned)(m & 0x3fffull));
                atomicAdd(&rx.hist[d * 4 + 2], (unsigned)((m >> 14) & 0x3fffull));
                atomicAdd(&rx.hist[d * 4 + 3], (unsigned)(m >> 28));
            }
        }
        __syncthreads();
        cluster_sync_all();
        // This CTA adds up its slice of the bins over the eight histograms ...
        unsigned long long c_bin = 0ull;
        unsigned long long m_bin = 0ull;
        if (tid < SLICE) {
            uint4 h[CS];
#pragma unroll
            for (uint32_t r = 0; r < CS; ++r) h[r] = ldc_v4(map_to_rank(smem_addr(&rx.hist[(rank * SLICE + tid) * 4]), r));
#pragma unroll
            for (uint32_t r = 0; r < CS; ++r) {
                c_bin += h[r].x;
                m_bin += (unsigned long long)h[r].y + ((unsigned long long)h[r].z << 14) + ((unsigned long long)h[r].w << 28);
            }
            s_cbin[tid] = c_bin;
            s_mbin[tid] = m_bin;
        }
        __syncthreads();
        if (tid < 32) {                                  // ... and shows the slice's totals to the others
            unsigned long long c = 0ull, m = 0ull;
#pragma unroll
            for (int j = 0; j < SLICE / 32; ++j) { c += s_cbin[tid * (SLICE / 32) + j]; m += s_mbin[tid * (SLICE / 32) + j]; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                c += __shfl_xor_sync(0xffffffffu, c, o);
                m += __shfl_xor_sync(0xffffffffu, m, o);
            }
            if (tid == 0) { rx.slice_cnt = c; rx.slice_mass = m; }
        }
        cluster_sync_all();
        // Walking the slices from the top, every CTA finds the slice in which the running total reaches
        // what is left; the CTA that owns it finds the bin and shows it.
        long long sc[CS];
        unsigned long long sm[CS];
#pragma unroll
        for (uint32_t r = 0; r < CS; ++r) {
            sc[r] = (long long)ldc_u64(map_to_rank(smem_addr(&rx.slice_cnt), r));
            sm[r] = ldc_u64(map_to_rank(smem_addr(&rx.slice_mass), r));
        }
        int own_k = -1, own_p = -1;
        unsigned long long c_above = 0ull;
        unsigned long long m_above = 0ull;
        {
            long long cr = 0;
            unsigned long long mr = 0ull;
#pragma unroll
            for (int r = CS - 1; r >= 0; --r) {
                if (own_k < 0 && cr + sc[r] >= k_left) { own_k = r; c_above = cr; }
                if (own_p < 0 && mr + sm[r] >= p_left) { own_p = r; m_above = mr; }
                cr += sc[r];
                mr += sm[r];
            }
        }
        if (tid < 32) {
            int digit;
            unsigned long long before;
            if (!k_done && own_k == (int)rank) {
                slice_crossing(s_cbin, c_above, (unsigned long long)k_left, digit, before);
                if (tid == 0) { rx.res_k_digit = rank * SLICE + digit; rx.res_k_before = before; }
            }
            if (!p_done && own_p == (int)rank) {
                slice_crossing(s_mbin, m_above, p_left, digit, before);
                if (tid == 0) { rx.res_p_digit = rank * SLICE + digit; rx.res_p_before = before; }
            }
        }
        cluster_sync_all();
        if (!k_done) {
            if (own_k >= 0) {
                thr_k |= (unsigned)ldc_s32(map_to_rank(smem_addr(&rx.res_k_digit), own_k)) << shift;
                k_left -= (long long)ldc_u64(map_to_rank(smem_addr(&rx.res_k_before), own_k));
            } else { thr_k = 0u; k_done = true; }        // fewer candidates than k: keep everything
        }
        if (!p_done) {
            if (own_p >= 0) {
                thr_p |= (unsigned)ldc_s32(map_to_rank(smem_addr(&rx.res_p_digit), own_p)) << shift;
                p_left -= ldc_u64(map_to_rank(smem_addr(&rx.res_p_before), own_p));
            } else { thr_p = 0u; p_done = true; }        // the whole mass stays below top-p: keep everything
        }
    }
    unsigned thr = thr_k > thr_p ? thr_k : thr_p;
    const float p_max = 1.0f * inv;                      // expf(0) * inv: the most probable token
    const float thr_m = min_p > 0.f ? min_p * p_max : 0.f;
    const unsigned b_max = __float_as_uint(p_max);
    if (thr > b_max) thr = b_max;                        // the most probable token always stays

    // ---- p^(1/T) over the kept set, renormalised (picolm/sampler.c:97-109)
    const float inv_t = 1.0f / temperature;
    float wsum = 0.f;
    for (int i = tid; i < n; i += NT) {
        const float p = prob[i];
        const bool keep = (__float_as_uint(p) >= thr) && (p >= thr_m || lo + i == best);
        const float w = keep ? __powf(p, inv_t) : 0.f;    // 2^(log2(p) / T) on the special-function unit
        prob[i] = w;
        wsum += w;
    }
    wsum = block_sum_f(wsum, redf);
    if (tid == 0) sh.sum = wsum;
    cluster_sync_all();
    float w_total = 0.f, w_before = 0.f;
    float ws[CS];
#pragma unroll
    for (uint32_t r = 0; r < CS; ++r) ws[r] = ldc_f32(map_to_rank(smem_addr(&sh.sum), r));
#pragma unroll
    for (uint32_t r = 0; r < CS; ++r) {
        if (r < rank) w_before += ws[r];
        w_total += ws[r];
    }
    const float inv_tot = w_total > 0.f ? 1.0f / w_total : 1.0f;

    // ---- the draw: first token, in index order, whose cumulative weight exceeds r
    unsigned long long x = rng[row_id];
    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
    const float rnd = (float)(x >> 11) / (float)(1ULL << 53);
    // every thread owns a run of consecutive tokens: its total, a scan of the totals over the block,
    // and the one thread whose run holds the crossing walks it
    __shared__ float seg_tot[NT];
    const int seg = ((n + NT - 1) / NT) | 1;             // odd: consecutive threads' runs fall into different banks
    const int s0 = min(n, tid * seg), s1 = min(n, s0 + seg);
    float mine = 0.f;
    for (int i = s0; i < s1; ++i) mine += prob[i] * inv_tot;
    seg_tot[tid] = mine;
    __syncthreads();
    if (tid < 32) {
        static_assert(NT == 256, "a lane of the first warp owns eight runs");
        float t8[8];
        float lane_tot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { t8[j] = seg_tot[tid * 8 + j]; lane_tot += t8[j]; }
        float incl = lane_tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, incl, o);
            if (tid >= o) incl += v;
        }
        float before = __shfl_up_sync(0xffffffffu, incl, 1);
        if (tid == 0) before = 0.f;
        const float start = w_before * inv_tot;
        const unsigned crossing = __ballot_sync(0xffffffffu, lane_tot > 0.f && start + incl > rnd);
        int chosen = INT_MAX;
        if (crossing && tid == __ffs(crossing) - 1) {
            float run = start + before;
            int last_seg = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) if (t8[j] > 0.f) last_seg = j;
            for (int j = 0; j < 8; ++j) {
                if (!(t8[j] > 0.f)) continue;
                if (run + t8[j] > rnd || j == last_seg) {
                    // the run that holds the crossing; where rounding lets the walk end below r, its last
                    // kept token is the one
                    const int o0 = min(n, (tid * 8 + j) * seg), o1 = min(n, o0 + seg);
                    for (int i = o0; i < o1; ++i) {
                        const float w = prob[i] * inv_tot;
                        if (!(w > 0.f)) continue;
                        run += w;
                        chosen = lo + i;
                        if (run > rnd) break;
                    }
                    break;
                }
                run += t8[j];
            }
        }
        if (crossing ? tid == __ffs(crossing) - 1 : tid == 0) sh.cand = chosen;
    }
    __syncthreads();

    cluster_sync_all();
    if (rank == 0 && tid == 0) {
        int c = INT_MAX;
        for (uint32_t r = 0; r < CS; ++r) c = min(c, ldc_s32(map_to_rank(smem_addr(&sh.cand), r)));
        out[row_id] = c == INT_MAX ? best : c;           // rounding left r above the total: the reference takes the top token
        rng[row_id] = x;
    }
    cluster_sync_all();
}

template <typename Kern, typename... Args>
int launch_cluster(Kern kern, int n_rows, size_t smem, cudaStream_t stream, Args... args) {
    return plm_status_of(launch_pdl_cluster(kern, dim3(n_rows * CS), dim3(NT), dim3(CS, 1, 1), smem, stream, args...));
}

int chunk_of(int V) { return ((V + CS - 1) / CS + 3) & ~3; }

}  // namespace

extern "C" int plm_argmax(const float* logits, long ld, int n_rows, int V, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (V <= 0 || ld < V) return PLM_ERR_SHAPE;
    return launch_cluster(argmax_kernel, n_rows, 0, stream, logits, ld, V, chunk_of(V), out);
}

// temperature > 0.  top_k <= 0 or >= V, top_p >= 1 and min_p <= 0 switch the respective cut off.
// rng holds one xorshift64 state per row (never 0).  Vocabularies beyond 8 * 40,960 entries are
// refused (a CTA keeps its eighth of the row in shared memory).
extern "C" int plm_sample(const float* logits, long ld, int n_rows, int V, float temperature, int top_k, float top_p,
                          float min_p, unsigned long long* rng, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (V <= 0 || ld < V) return PLM_ERR_SHAPE;
    if (!(temperature > 0.f)) return PLM_ERR_UNSUPPORTED;
    const int chunk = chunk_of(V);
    if (chunk > MAX_CHUNK) return PLM_ERR_UNSUPPORTED;
    const size_t smem = (size_t)chunk * sizeof(float);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        const size_t most = MAX_CHUNK * sizeof(float);
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess) return (int)e;
        configured = most;
    }
    return launch_cluster(sample_kernel, n_rows, smem, stream, logits, ld, V, chunk, temperature, top_k, top_p, min_p, rng,
                          out);
}
