// Causal attention of new tokens over the paged cache, one warp per
// (token, query head), on the CUDA cores with fp32 arithmetic throughout.
//
// For a query at absolute position p with head h, KV head g = h / (H / G):
//   s_t = (q_h . K[t, g]) * scale  for t in [lo, p],  out_h = softmax(s) . V[:, g]
// with the running (max, sum, acc) update of the reference's `attn_core`
// (picolm/model_attention.c:43-140; max starts at -1e30, causal by the loop
// bound) taken 32 keys at a time.  lo = 0, or p - window + 1 for a sliding
// window.  Keys and values of position t of sequence b live at
//   cache[block_table[b][t / PLM_PAGE]][g][t % PLM_PAGE][0..hd)
// and the new tokens' own K/V are already there when this kernel runs.
//
// This is the attention of the float32 path, and the any-size attention of the
// bfloat16 path (head sizes that the tensor-core kernels refuse).  A row's
// result depends on its own position and sequence only.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;            // acc registers per lane: MAX_HD / 32

template <typename Ta, typename Tc>
__global__ void __launch_bounds__(WARPS * 32)
attention_rows_kernel(const Ta* __restrict__ q, const Tc* __restrict__ kc, const Tc* __restrict__ vc,
                      Ta* __restrict__ out, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                      const int* __restrict__ block_table, int max_pages, int H, int G, int hd, float scale,
                      int window) {
    extern __shared__ float q_sm[];                 // [WARPS][hd]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= H) return;                             // warp-level exit; no block barrier below
    const int g = h / (H / G);
    const int pos = PLM_POSITION(tok_pos[t]);
    const int* pages = block_table + (size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages;
    float* qs = q_sm + warp * hd;
    const Ta* qrow = q + ((size_t)t * H + h) * hd;
    for (int i = lane; i < hd; i += 32) qs[i] = to_f32<Ta>(qrow[i]);
    __syncwarp();

    float acc[MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;
    float m = -1e30f, l = 0.f;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    for (int base = lo; base <= pos; base += 32) {
        const int key = base + lane;
        float s = -1e30f;
        const bool valid = key <= pos;
        if (valid) {
            const int page = PLM_PAGE_NO(pages[key / PLM_PAGE]);
            const Tc* kr = kc + (((size_t)page * G + g) * PLM_PAGE + key % PLM_PAGE) * hd;
            float dot = 0.f;
            for (int i = 0; i < hd; ++i) dot = fmaf(qs[i], to_f32<Tc>(kr[i]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
        const int n_keys = min(32, pos - base + 1);
        for (int j = 0; j < n_keys; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const int kj = base + j;
            const int page = PLM_PAGE_NO(pages[kj / PLM_PAGE]);
            const Tc* vr = vc + (((size_t)page * G + g) * PLM_PAGE + kj % PLM_PAGE) * hd;
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_f32<Tc>(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
    Ta* o = out + ((size_t)t * H + h) * hd;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = from_f32<Ta>(acc[i] * inv);
    }
}

}  // namespace

// q [T, H, hd] and out [T, H, hd] have the activation type, the cache its own;
// both are PLM_F32 or both PLM_BF16.
extern "C" int plm_attention_rows(const void* q, const void* kc, const void* vc, void* out, int dtype,
                                  const int* tok_pos, const int* tok_seq, const int* block_table, int max_pages,
                                  int n_tokens, int H, int G, int hd, float scale, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || H % G || hd <= 0 || hd > MAX_HD) return PLM_ERR_SHAPE;
    dim3 grid(n_tokens, (H + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    if (dtype == PLM_F32)
        attention_rows_kernel<float, float><<<grid, WARPS * 32, smem, stream>>>(
            (const float*)q, (const float*)kc, (const float*)vc, (float*)out, tok_pos, tok_seq, block_table, max_pages,
            H, G, hd, scale, window);
    else if (dtype == PLM_BF16)
        attention_rows_kernel<bf16, bf16><<<grid, WARPS * 32, smem, stream>>>(
            (const bf16*)q, (const bf16*)kc, (const bf16*)vc, (bf16*)out, tok_pos, tok_seq, block_table, max_pages, H,
            G, hd, scale, window);
    else
        return PLM_ERR_DTYPE;
    return plm_launch_status();
}
