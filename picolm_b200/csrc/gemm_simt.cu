// C[M,N] = A[M,K] * W[N,K]^T with fp32 accumulation on the CUDA cores.
//
// This is the reference's `matmul(out, x, W, n, d)`: W is row-major
// [out_features, in_features] and every output is the dot product of one weight
// row with the input (picolm/tensor.c:1394-1418), element types widened to fp32
// inside the dot product (picolm/quant.c:133-153, picolm/quant.c:679).
//
// It is the matrix product of the float32 path (plain FFMA, no reduced-precision
// matrix mode) and the any-size product of the bfloat16 path when a shape does
// not fit the tensor-core kernel.  Each output element is accumulated over k in
// ascending order by one thread, so a row's result never depends on which other
// rows are in the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

template <typename Ta, typename Tw, typename To>
__global__ void __launch_bounds__(NT)
gemm_simt_kernel(const Ta* __restrict__ A, const Tw* __restrict__ W, To* __restrict__ C, int M, int N, int K,
                 long lda, long ldw, long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int ty = tid / 16, tx = tid % 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int it = 0; it < (BM * BK) / NT; ++it) {
            const int idx = tid + it * NT;
            const int r = idx / BK, k = idx % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? to_f32<Ta>(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[k][r] = (gn < N && gk < K) ? to_f32<Tw>(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_f32<To>(acc[i][j]);
        }
    }
}

template <typename Ta, typename Tw, typename To>
int launch(const void* A, const void* W, void* C, int M, int N, int K, long lda, long ldw, long ldc,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_simt_kernel<Ta, Tw, To><<<grid, NT, 0, stream>>>((const Ta*)A, (const Tw*)W, (To*)C, M, N, K, lda, ldw, ldc);
    return plm_launch_status();
}

}  // namespace

// Leading dimensions are in elements.  Supported (A, W, C) element types:
// (f32,f32,f32), (bf16,bf16,bf16|f32), (bf16,f32,bf16|f32).
extern "C" int plm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N,
                             int K, long lda, long ldw, long ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return PLM_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return PLM_ERR_SHAPE;
    if ((M + BM - 1) / BM > 65535) return PLM_ERR_SHAPE;
    if (a_dtype == PLM_F32 && w_dtype == PLM_F32 && c_dtype == PLM_F32)
        return launch<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    if (a_dtype == PLM_BF16 && w_dtype == PLM_BF16 && c_dtype == PLM_BF16)
        return launch<bf16, bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    if (a_dtype == PLM_BF16 && w_dtype == PLM_BF16 && c_dtype == PLM_F32)
        return launch<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    if (a_dtype == PLM_BF16 && w_dtype == PLM_F32 && c_dtype == PLM_BF16)
        return launch<bf16, float, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    if (a_dtype == PLM_BF16 && w_dtype == PLM_F32 && c_dtype == PLM_F32)
        return launch<bf16, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    return PLM_ERR_DTYPE;
}
