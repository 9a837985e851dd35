// Row-wise and element-wise kernels of the decoder: token embedding gather,
// RMSNorm with the residual add folded in, SwiGLU, and rotary position
// encoding fused with the write of K and V into the paged cache.
//
// Formulas follow the reference's scalar forms:
//   RMSNorm   ss = sum x^2; r = 1/sqrtf(ss/size + eps); out = (x*r)*w   (picolm/tensor.c:2942-3064)
//   SiLU      x / (1 + expf(-x)), multiplied by the up branch             (picolm/tensor.c:3306-3315,
//                                                                          picolm/model_core.c:2192-2193)
//   RoPE      (x0,x1) -> (x0*c - x1*s, x0*s + x1*c), q and k only         (picolm/tensor.c:3216-3304)
//   embedding x = float(row of the table), no scale                       (picolm/model_core.c:1785-1786)
// All statistics and the residual stream are fp32.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename Tw>
__global__ void embed_kernel(const int* __restrict__ tok, const Tw* __restrict__ table, float* __restrict__ out,
                             int d, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = tok[t];
    if (id < 0 || id >= vocab) id = 0;   // ids are checked on the host; never read outside the table
    const Tw* row = table + (size_t)id * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<Tw>(row[i]);
}

extern "C" int plm_embed(const int* tok, const void* table, int table_dtype, float* out, int n_tokens, int d,
                         int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (d <= 0 || vocab <= 0) return PLM_ERR_SHAPE;
    const int nt = d >= 1024 ? 256 : 128;
    if (table_dtype == PLM_F32)
        return plm_status_of(launch_pdl(embed_kernel<float>, n_tokens, nt, 0, stream, tok, (const float*)table, out, d, vocab));
    if (table_dtype == PLM_BF16)
        return plm_status_of(launch_pdl(embed_kernel<bf16>, n_tokens, nt, 0, stream, tok, (const bf16*)table, out, d, vocab));
    return PLM_ERR_DTYPE;
}

// -------------------------------------------------------------------- RMSNorm
// One block per output row.  Row r reads source row rows[r] (or r).  With a
// delta the sum x + delta is normalised; it is written back to x unless rows are
// gathered.  The reduction order depends on the row's width only, never on what
// else is in the batch.

template <typename Tw, typename To, int NT>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const Tw* __restrict__ w,
                               To* __restrict__ out, const int* __restrict__ rows, int d, float eps, int write_back) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NT) {
        float v = xr[i];
        if (dr) {
            v += dr[i];
            if (write_back) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum<NT>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    To* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += NT) {
        float v = xr[i];
        if (dr && !write_back) v += dr[i];
        o[i] = from_f32<To>(v * scale * to_f32<Tw>(w[i]));
    }
}

// Four elements at a time, the row kept in registers between the two passes: for rows whose width
// is a multiple of 4 and at most 16 * NT.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename Tw, typename To, int NT>
__global__ void __launch_bounds__(NT)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, const Tw* __restrict__ w,
                   To* __restrict__ out, const int* __restrict__ rows, int d, float eps, int write_back) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            v[k] = load4(xr + i);
            if (dr) {
                const float4 dv = load4(dr + i);
                v[k].x += dv.x; v[k].y += dv.y; v[k].z += dv.z; v[k].w += dv.w;
                if (write_back) store4(xr + i, v[k]);
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum<NT>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    To* o = out + (size_t)r * d;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            const float4 wv = load4(w + i);
            store4(o + i, make_float4(v[k].x * scale * wv.x, v[k].y * scale * wv.y, v[k].z * scale * wv.z,
                                      v[k].w * scale * wv.w));
        }
    }
}

template <typename Tw, typename To>
static int rmsnorm_launch(float* x, const float* delta, const void* w, void* out, const int* rows, int n_rows, int d,
                          float eps, int write_back, cudaStream_t stream) {
    if (d % 4 == 0 && d <= 16 * 1024) {
        // the block size (and with it the order of the sum of squares) depends on the row's width only
        if (d <= 16 * 256)
            return plm_status_of(launch_pdl(rmsnorm_vec_kernel<Tw, To, 256>, n_rows, 256, 0, stream, x, delta,
                                            (const Tw*)w, (To*)out, rows, d, eps, write_back));
        return plm_status_of(launch_pdl(rmsnorm_vec_kernel<Tw, To, 1024>, n_rows, 1024, 0, stream, x, delta,
                                        (const Tw*)w, (To*)out, rows, d, eps, write_back));
    }
    // enough threads that a row's loads are all in flight at once; the block size (and with it the
    // order of the sum of squares) depends on the row's width only
    if (d > 1024)
        return plm_status_of(launch_pdl(rmsnorm_kernel<Tw, To, 1024>, n_rows, 1024, 0, stream, x, delta,
                                        (const Tw*)w, (To*)out, rows, d, eps, write_back));
    return plm_status_of(launch_pdl(rmsnorm_kernel<Tw, To, 256>, n_rows, 256, 0, stream, x, delta, (const Tw*)w,
                                    (To*)out, rows, d, eps, write_back));
}

extern "C" int plm_rmsnorm(float* x, const float* delta, const void* w, int w_dtype, void* out, int out_dtype,
                           const int* rows, int n_rows, int d, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0) return PLM_ERR_SHAPE;
    const int write_back = (delta != nullptr && rows == nullptr) ? 1 : 0;
    if (w_dtype == PLM_F32 && out_dtype == PLM_F32)
        return rmsnorm_launch<float, float>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_F32)
        return rmsnorm_launch<bf16, float>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_F32 && out_dtype == PLM_BF16)
        return rmsnorm_launch<float, bf16>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_BF16)
        return rmsnorm_launch<bf16, bf16>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------ rows whose scale is still due
// out[t, :] = bf16(x[t, :] * r[t]) with r[t] = 1 / sqrt(sum_p parts[p, t] / size + eps): what is left of
// an RMSNorm whose weight a product's epilogue has already applied (x) and whose sums of squares it has
// left as partial sums (parts [n_parts, ld_parts]).  One block per row, sums in a fixed order.
__global__ void scale_rows_kernel(const bf16* __restrict__ x, const float* __restrict__ parts, int n_parts, int ld_parts,
                                  float inv_size, float eps, bf16* __restrict__ out, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int p = 0; p < n_parts; ++p) ss += parts[(size_t)p * ld_parts + t];
    const float r = 1.0f / sqrtf(ss * inv_size + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[(size_t)t * d + i] = __float2bfloat16_rn(__bfloat162float(x[(size_t)t * d + i]) * r);
}

extern "C" int plm_scale_rows(const void* x, const float* parts, int n_parts, int ld_parts, int size, float eps,
                              void* out, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0 || size <= 0 || n_parts <= 0 || ld_parts < n_rows) return PLM_ERR_SHAPE;
    return plm_status_of(launch_pdl(scale_rows_kernel, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, parts, n_parts,
                                    ld_parts, 1.0f / (float)size, eps, (bf16*)out, d));
}

// ----------------------------------------------------------- gated activation
// gu is [T, 2F]: gate in columns [0,F), up in [F,2F).  out[T,F] = act(gate) * up, with
// ACT 0: silu(g) = g / (1 + expf(-g))                                  (picolm/tensor.c:3306-3315)
// ACT 1: gelu(g) = 0.5 g (1 + tanhf(0.79788456 (g + 0.044715 g^3)))    (picolm/tensor.c:3317-3323)
template <int ACT> __device__ __forceinline__ float gate_act(float g);
template <> __device__ __forceinline__ float gate_act<0>(float g) { return g / (1.0f + expf(-g)); }
template <> __device__ __forceinline__ float gate_act<1>(float g) {
    return 0.5f * g * (1.0f + tanhf(0.79788456f * (g + 0.044715f * g * g * g)));
}

template <typename T, int ACT>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t t = i / F;
        const int c = (int)(i - t * F);
        const float g = to_f32<T>(gu[t * 2 * F + c]);
        const float u = to_f32<T>(gu[t * 2 * F + F + c]);
        out[i] = from_f32<T>(gate_act<ACT>(g) * u);
    }
}

template <typename T>
static int launch_gated(int act, int blocks, cudaStream_t stream, const T* gu, T* out, int F, size_t total) {
    if (act == 0) return plm_status_of(launch_pdl(swiglu_kernel<T, 0>, blocks, 256, 0, stream, gu, out, F, total));
    if (act == 1) return plm_status_of(launch_pdl(swiglu_kernel<T, 1>, blocks, 256, 0, stream, gu, out, F, total));
    return PLM_ERR_UNSUPPORTED;
}

// act: 0 silu, 1 gelu (tanh form)
extern "C" int plm_swiglu(const void* gu, void* out, int dtype, int act, int n_rows, int F, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (F <= 0) return PLM_ERR_SHAPE;
    const size_t total = (size_t)n_rows * F;
    int blocks = (int)((total + 255) / 256);
    if (blocks > PLM_SM_COUNT * 16) blocks = PLM_SM_COUNT * 16;
    if (dtype == PLM_F32) return launch_gated<float>(act, blocks, stream, (const float*)gu, (float*)out, F, total);
    if (dtype == PLM_BF16) return launch_gated<bf16>(act, blocks, stream, (const bf16*)gu, (bf16*)out, F, total);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------- RoPE + write into the cache
// qkv is [T, (H + 2G) * hd]: H query heads, then G key heads, then G value heads.
// Query heads are rotated into q_out [T, H, hd]; key heads are rotated and
// written, value heads copied, into the paged cache
//   cache[page][g][slot_in_page][hd],  page = block_table[seq][pos / PLM_PAGE].
// cos/sin are [table_len, rot_dim/2] fp32 tables; null tables mean no rotation.
// pairing 0: (x[i], x[i + rot_dim/2]); pairing 1: (x[2i], x[2i+1]).  Elements at
// and beyond rot_dim pass through.  store = 0 skips the cache (a layer that reads
// another layer's cache).
template <typename Ta, typename Tc>
__global__ void rope_store_kernel(const Ta* __restrict__ qkv, Ta* __restrict__ q_out, Tc* __restrict__ kc,
                                  Tc* __restrict__ vc, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                  int max_pages, int H, int G, int hd, int rot_dim, int pairing, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = PLM_POSITION(tok_pos[t]);
    const int half = hd / 2, rot_half = rot_dim / 2;
    const int n_heads = H + 2 * G;
    const Ta* row = qkv + (size_t)t * n_heads * hd;
    size_t page_base = 0;
    int in_page = 0;
    bool have_page = false;
    if (store) {
        const int page = PLM_PAGE_NO(block_table[(size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages + pos / PLM_PAGE]);
        have_page = page >= 0;
        page_base = (size_t)(page < 0 ? 0 : page) * G;
        in_page = pos % PLM_PAGE;
    }
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_heads * half; item += gridDim.y * blockDim.x) {
        const int head = item / half, j = item - head * half;
        int ia, ib;
        bool rotate = (j < rot_half) && cos_t != nullptr;
        if (j < rot_half) {
            if (pairing == 0) { ia = j; ib = j + rot_half; } else { ia = 2 * j; ib = 2 * j + 1; }
        } else {
            ia = rot_dim + 2 * (j - rot_half); ib = ia + 1;
        }
        float a = to_f32<Ta>(row[head * hd + ia]);
        float b = to_f32<Ta>(row[head * hd + ib]);
        if (head < H) {
            if (rotate) {
                const float c = cos_t[(size_t)pos * rot_half + j], s = sin_t[(size_t)pos * rot_half + j];
                const float ra = rope_first(a, b, c, s), rb = rope_second(a, b, c, s);
                a = ra; b = rb;
            }
            Ta* o = q_out + ((size_t)t * H + head) * hd;
            o[ia] = from_f32<Ta>(a);
            o[ib] = from_f32<Ta>(b);
        } else if (head < H + G) {
            if (!store || !have_page) continue;
            if (rotate) {
                const float c = cos_t[(size_t)pos * rot_half + j], s = sin_t[(size_t)pos * rot_half + j];
                const float ra = rope_first(a, b, c, s), rb = rope_second(a, b, c, s);
                a = ra; b = rb;
            }
            const int g = head - H;
            Tc* o = kc + ((page_base + g) * PLM_PAGE + in_page) * hd;
            o[ia] = from_f32<Tc>(a);
            o[ib] = from_f32<Tc>(b);
        } else {
            if (!store || !have_page) continue;
            const int g = head - H - G;
            Tc* o = vc + ((page_base + g) * PLM_PAGE + in_page) * hd;
            o[ia] = from_f32<Tc>(a);
            o[ib] = from_f32<Tc>(b);
        }
    }
}

// The common case eight pairs at a time: bf16, the whole head rotated (rot_dim == hd), half-split
// pairing, head size a multiple of 16.  A thread takes x[j..j+8) and x[half+j..half+j+8) of one head
// as two 16-byte loads and writes two 16-byte stores.
__global__ void rope_store_vec_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ kc,
                                      bf16* __restrict__ vc, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                      int max_pages, int H, int G, int hd, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = PLM_POSITION(tok_pos[t]);
    const int half = hd / 2, groups = half / 8;
    const int n_heads = H + 2 * G;
    const bf16* row = qkv + (size_t)t * n_heads * hd;
    size_t page_base = 0;
    int in_page = 0;
    bool have_page = false;
    if (store) {
        const int page = PLM_PAGE_NO(block_table[(size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages + pos / PLM_PAGE]);
        have_page = page >= 0;
        page_base = (size_t)(page < 0 ? 0 : page) * G;
        in_page = pos % PLM_PAGE;
    }
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_heads * groups; item += gridDim.y * blockDim.x) {
        const int head = item / groups, j = (item - head * groups) * 8;
        bf16* dst;
        if (head < H) {
            dst = q_out + ((size_t)t * H + head) * hd;
        } else {
            if (!store || !have_page) continue;
            const int g = head < H + G ? head - H : head - H - G;
            dst = (head < H + G ? kc : vc) + ((page_base + g) * PLM_PAGE + in_page) * hd;
        }
        uint4 lo = *reinterpret_cast<const uint4*>(row + head * hd + j);
        uint4 hi = *reinterpret_cast<const uint4*>(row + head * hd + half + j);
        if (head < H + G) {
            const float4 c0 = load4(cos_t + (size_t)pos * half + j), c1 = load4(cos_t + (size_t)pos * half + j + 4);
            const float4 s0 = load4(sin_t + (size_t)pos * half + j), s1 = load4(sin_t + (size_t)pos * half + j + 4);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a0 = __low2float(l2[k]), a1 = __high2float(l2[k]);
                const float b0 = __low2float(h2[k]), b1 = __high2float(h2[k]);
                l2[k] = __floats2bfloat162_rn(rope_first(a0, b0, c[2 * k], sn[2 * k]), rope_first(a1, b1, c[2 * k + 1], sn[2 * k + 1]));
                h2[k] = __floats2bfloat162_rn(rope_second(a0, b0, c[2 * k], sn[2 * k]), rope_second(a1, b1, c[2 * k + 1], sn[2 * k + 1]));
            }
        }
        *reinterpret_cast<uint4*>(dst + j) = lo;
        *reinterpret_cast<uint4*>(dst + half + j) = hi;
    }
}

extern "C" int plm_rope_store(const void* qkv, void* q_out, void* kc, void* vc, int dtype, const float* cos_t,
                              const float* sin_t, const int* tok_pos, const int* tok_seq, const int* block_table,
                              int max_pages, int n_tokens, int H, int G, int hd, int rot_dim, int pairing, int store,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || hd <= 0 || (hd & 1) || rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return PLM_ERR_SHAPE;
    if (pairing != 0 && pairing != 1) return PLM_ERR_UNSUPPORTED;
    if (dtype == PLM_BF16 && pairing == 0 && rot_dim == hd && hd % 16 == 0 && cos_t != nullptr) {
        const int vitems = (H + 2 * G) * (hd / 16);
        int vchunks = (vitems + 127) / 128;
        if (vchunks > 64) vchunks = 64;
        return plm_status_of(launch_pdl(rope_store_vec_kernel, dim3(n_tokens, vchunks), dim3(128), 0, stream,
                                        (const bf16*)qkv, (bf16*)q_out, (bf16*)kc, (bf16*)vc, cos_t, sin_t, tok_pos,
                                        tok_seq, block_table, max_pages, H, G, hd, store));
    }
    const int items = (H + 2 * G) * (hd / 2);
    const int nt_threads = items >= 128 ? 128 : 64;
    int chunks = (items + nt_threads - 1) / nt_threads;
    if (chunks > 64) chunks = 64;
    const dim3 nt(nt_threads), grid_rs(n_tokens, chunks);
    if (dtype == PLM_F32)
        return plm_status_of(launch_pdl(rope_store_kernel<float, float>, grid_rs, nt, 0, stream, (const float*)qkv,
                                        (float*)q_out, (float*)kc, (float*)vc, cos_t, sin_t, tok_pos,
                                        tok_seq, block_table, max_pages, H, G, hd, rot_dim, pairing, store));
    if (dtype == PLM_BF16)
        return plm_status_of(launch_pdl(rope_store_kernel<bf16, bf16>, grid_rs, nt, 0, stream, (const bf16*)qkv,
                                        (bf16*)q_out, (bf16*)kc, (bf16*)vc, cos_t, sin_t, tok_pos,
                                        tok_seq, block_table, max_pages, H, G, hd, rot_dim, pairing, store));
    return PLM_ERR_DTYPE;
}

// dst[i, :] = src[rows[i], :] for rows of `row_bytes` bytes (a multiple of 4; 16 bytes at a time where the rows
// and both pointers allow it).  Rows of a prompt step that are wanted further on, out of all of its rows.
__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int* __restrict__ rows,
                                   long row_bytes, long src_ld, int wide) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const uint8_t* s = src + (size_t)PLM_ROW_NO(rows[i]) * src_ld;
    uint8_t* d = dst + (size_t)i * row_bytes;
    if (wide) {
        for (long o = (long)threadIdx.x * 16; o < row_bytes; o += (long)blockDim.x * 16)
            *reinterpret_cast<uint4*>(d + o) = *reinterpret_cast<const uint4*>(s + o);
    } else {
        for (long o = (long)threadIdx.x * 4; o < row_bytes; o += (long)blockDim.x * 4)
            *reinterpret_cast<uint32_t*>(d + o) = *reinterpret_cast<const uint32_t*>(s + o);
    }
}

extern "C" int plm_gather_rows(const void* src, void* dst, const int* rows, int n_rows, long row_bytes, long src_ld_bytes,
                               cudaStream_t stream) {
    if (n_rows <= 0 || row_bytes <= 0) return PLM_OK;
    if (row_bytes % 4 || src_ld_bytes % 4 || (((uintptr_t)src | (uintptr_t)dst) & 3)) return PLM_ERR_ALIGN;
    const int wide = row_bytes % 16 == 0 && src_ld_bytes % 16 == 0 && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0);
    return plm_status_of(launch_pdl(gather_rows_kernel, dim3(n_rows), dim3(256), 0, stream, (const uint8_t*)src,
                                    (uint8_t*)dst, rows, row_bytes, src_ld_bytes, wide));
}
