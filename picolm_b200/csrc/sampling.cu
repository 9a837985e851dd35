// Token selection from fp32 logits on the device: greedy argmax and the
// reference's sampling chain softmax -> top-k -> top-p -> min-p -> p^(1/T) -> draw
// (picolm/sampler.c:48-125), one thread block per sequence.
//
// The reference sorts the probabilities and cuts the sorted list; a cut of a
// sorted list is the set {p >= threshold}, so the kept set is found here without
// a sort, by raising a threshold bit by bit while the kept count (top-k) or the
// kept mass (top-p) still reaches its target.  Values that tie with the value at
// the cut are all kept.  The draw walks the kept tokens in index order (the
// reference walks them in sorted order): the same distribution, another token for
// a given random number.  Random numbers are the reference's xorshift64 stream
// (picolm/sampler.c:10-21), one state per sequence, advanced in place.
// All sums are tree reductions in a fixed order: same inputs, same token.
#include "common.cuh"
#include <limits.h>

namespace {

constexpr int NT = 1024;

__device__ __forceinline__ float block_max_f(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = red[lane];
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ int block_sum_i(int v, int* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ int block_min_i(int v, int* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// First index of the maximum (strict > scan from index 0, picolm/sampler.c:50-56).
__device__ int block_argmax(const float* __restrict__ row, int V, float* redf, int* redi) {
    float best = -INFINITY;
    int idx = INT_MAX;
    for (int i = threadIdx.x; i < V; i += NT) {
        const float v = row[i];
        if (v > best) { best = v; idx = i; }        // ascending i per thread: first index wins ties
    }
    const float m = block_max_f(best, redf);
    const int cand = (best == m && idx != INT_MAX) ? idx : INT_MAX;
    const int r = block_min_i(cand, redi);
    return r == INT_MAX ? 0 : r;
}

__global__ void __launch_bounds__(NT) argmax_kernel(const float* __restrict__ logits, long ld, int V,
                                                    int* __restrict__ out) {
    __shared__ float redf[33];
    __shared__ int redi[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = block_argmax(logits + (size_t)blockIdx.x * ld, V, redf, redi);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, long ld, int V, float temperature, int top_k, float top_p, float min_p,
              unsigned long long* __restrict__ rng, int* __restrict__ out) {
    __shared__ float redf[33];
    __shared__ int redi[33];
    __shared__ float warp_tot[32];
    __shared__ float s_r;
    const float* row = logits + (size_t)blockIdx.x * ld;
    const int tid = threadIdx.x;

    const int best = block_argmax(row, V, redf, redi);
    const float mx = row[best];
    float z = 0.f;
    for (int i = tid; i < V; i += NT) z += expf(row[i] - mx);
    z = block_sum<NT>(z, redf);
    const float inv = 1.0f / z;
    // p_i = expf(l_i - max) * inv, recomputed wherever it is needed (picolm/tensor.c:3066-3076)

    const bool use_k = top_k > 0 && top_k < V;
    unsigned thr_k = 0u, thr_p = 0u;
    for (int bit = 30; bit >= 0; --bit) {
        const unsigned ck = thr_k | (1u << bit), cp = thr_p | (1u << bit);
        int cnt = 0;
        float mass = 0.f;
        for (int i = tid; i < V; i += NT) {
            const float p = expf(row[i] - mx) * inv;
            const unsigned b = __float_as_uint(p);
            if (use_k && b >= ck) ++cnt;
            if (b >= cp) mass += p;
        }
        if (use_k) {
            cnt = block_sum_i(cnt, redi);
            if (cnt >= top_k) thr_k = ck;
        }
        mass = block_sum<NT>(mass, redf);
        if (mass >= top_p) thr_p = cp;
    }
    unsigned thr = thr_k > thr_p ? thr_k : thr_p;
    const float p_max = 1.0f * inv;                       // expf(0) * inv
    const float thr_m = min_p > 0.f ? min_p * p_max : 0.f;
    const unsigned b_max = __float_as_uint(p_max);
    if (thr > b_max) thr = b_max;                         // the most probable token always stays

    // p^(1/T), renormalised over the kept set (picolm/sampler.c:97-109)
    const float inv_t = 1.0f / temperature;
    float tot = 0.f;
    for (int i = tid; i < V; i += NT) {
        const float p = expf(row[i] - mx) * inv;
        const bool keep = (__float_as_uint(p) >= thr) && (p >= thr_m || i == best);
        if (keep) tot += powf(p, inv_t);
    }
    tot = block_sum<NT>(tot, redf);
    const float inv_tot = tot > 0.f ? 1.0f / tot : 1.0f;

    if (tid == 0) {
        unsigned long long x = rng[blockIdx.x];
        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
        rng[blockIdx.x] = x;
        s_r = (float)(x >> 11) / (float)(1ULL << 53);
    }
    __syncthreads();
    const float r = s_r;

    // inverse CDF in index order: first i with cumulative > r
    const int lane = tid & 31, warp = tid >> 5;
    float running = 0.f;
    int chosen = INT_MAX;
    for (int base = 0; base < V; base += NT) {
        const int i = base + tid;
        float w = 0.f;
        if (i < V) {
            const float p = expf(row[i] - mx) * inv;
            const bool keep = (__float_as_uint(p) >= thr) && (p >= thr_m || i == best);
            if (keep) w = powf(p, inv_t) * inv_tot;
        }
        float s = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float u = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += u;
        }
        __syncthreads();
        if (lane == 31) warp_tot[warp] = s;
        __syncthreads();
        float before = 0.f;
        for (int wi = 0; wi < warp; ++wi) before += warp_tot[wi];
        const float cum = running + before + s;
        int cand = (w > 0.f && cum > r) ? i : INT_MAX;
        cand = block_min_i(cand, redi);
        if (cand != INT_MAX) { chosen = cand; break; }     // uniform across the block
        float chunk = 0.f;
        for (int wi = 0; wi < NT / 32; ++wi) chunk += warp_tot[wi];
        running += chunk;
    }
    if (tid == 0) out[blockIdx.x] = (chosen == INT_MAX) ? best : chosen;
}

}  // namespace

extern "C" int plm_argmax(const float* logits, long ld, int n_rows, int V, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (V <= 0 || ld < V) return PLM_ERR_SHAPE;
    return plm_status_of(launch_pdl(argmax_kernel, dim3(n_rows), dim3(NT), 0, stream, logits, ld, V, out));
}

// temperature > 0.  top_k <= 0 or >= V, top_p >= 1 and min_p <= 0 switch the
// respective cut off.  rng holds one xorshift64 state per row (never 0).
extern "C" int plm_sample(const float* logits, long ld, int n_rows, int V, float temperature, int top_k, float top_p,
                          float min_p, unsigned long long* rng, int* out, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (V <= 0 || ld < V) return PLM_ERR_SHAPE;
    if (!(temperature > 0.f)) return PLM_ERR_UNSUPPORTED;
    sample_kernel<<<n_rows, NT, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p, rng, out);
    return plm_launch_status();
}
