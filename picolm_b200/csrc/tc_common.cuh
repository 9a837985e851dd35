// Building blocks shared by the tcgen05 matrix-product kernels: mbarrier and TMA wrappers with
// bounded waits, tcgen05 (MMA, commit, TMEM load) wrappers, the shared-memory and instruction
// descriptors of a K-major bf16 tile with 128-byte swizzle, and the host-side tensor map.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <mutex>

namespace plm_tc {

constexpr int BM = 128;                  // rows of P per tile (TMEM lanes)
constexpr int BK = 64;                   // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
#ifndef PLM_WAIT_LIMIT
#define PLM_WAIT_LIMIT (1u << 24)        // a test build shortens it so that a wait that runs out does so at once
#endif
constexpr uint32_t WAIT_LIMIT = PLM_WAIT_LIMIT;   // polls of mbarrier.try_wait before giving up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `where`) if the phase did not complete.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int where) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicCAS(status, 0, where);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// rows from `row`, all 64 columns, slabs of K from `slab`: a map of make_map with slabs > 1
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row, int slab) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(0), "r"(row), "r"(slab) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes
// (64 elements) with the 128-byte swizzle that TMA wrote: 8-row groups are 1024
// bytes apart (SBO), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// silu(g) * u for the fused bf16 epilogues: g and u are rounded to bf16 first (as a separate
// activation kernel would read them), then g / (1 + 2^(-g log2 e)) * u with the special-function
// unit's 2^x and reciprocal, whose error is far below the bf16 rounding of the result.
// Wait for the tensor-memory loads in flight, of which `r` (32 registers) is a destination: the registers count as
// written here, so that nothing the compiler makes of them moves above the wait.
__device__ __forceinline__ void tc_wait_ld_into(uint32_t* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(r[i]));
}

__device__ __forceinline__ float swiglu_bf16(float g, float u) {
    g = __bfloat162float(__float2bfloat16_rn(g));
    u = __bfloat162float(__float2bfloat16_rn(u));
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    return __fdividef(g, 1.0f + e) * u;
}

template <typename T> __device__ __forceinline__ void store_vec8(T* p, const uint32_t* r);
template <> __device__ __forceinline__ void store_vec8<float>(float* p, const uint32_t* r) {
    reinterpret_cast<uint4*>(p)[0] = make_uint4(r[0], r[1], r[2], r[3]);
    reinterpret_cast<uint4*>(p)[1] = make_uint4(r[4], r[5], r[6], r[7]);
}
template <> __device__ __forceinline__ void store_vec8<bf16>(bf16* p, const uint32_t* r) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bf16 row-major matrix with leading dimension ld (elements); boxes of box_rows x 64.
// With `slabs` > 1 (K a multiple of 64) the matrix is described as [K / 64 slabs][rows][64] and a box holds
// `slabs` consecutive slabs of box_rows x 64: one copy brings in what `slabs` copies of the plain form do, and
// lands as that many tiles one behind the other.  (A tensor copy occupies an SM's copy engine for some 300
// cycles whatever its size, so a kernel bound by its copies wants few and large ones.)
// Descriptors are kept in a small table by what they describe (a descriptor depends on nothing else, and
// encoding one costs a few microseconds of host time per operand and launch).
static inline int make_map(CUtensorMap* map, const void* ptr, long rows, long K, long ld, int box_rows, int slabs = 1) {
    struct Entry { const void* ptr; long rows, K, ld; int box_rows, slabs; bool used; CUtensorMap map; };
    constexpr int SLOTS = 512;
    static Entry table[SLOTS];
    static std::mutex lock;
    if (slabs < 1 || (slabs > 1 && K % BK)) return PLM_ERR_SHAPE;
    const size_t h = ((size_t)ptr >> 4) * 0x9E3779B97F4A7C15ull + (size_t)rows * 31 + (size_t)K * 131 + (size_t)box_rows +
                     (size_t)slabs * 7919;
    Entry& e = table[(h >> 20) % SLOTS];
    {
        std::lock_guard<std::mutex> g(lock);
        if (e.used && e.ptr == ptr && e.rows == rows && e.K == K && e.ld == ld && e.box_rows == box_rows && e.slabs == slabs) {
            *map = e.map;
            return PLM_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return PLM_ERR_UNSUPPORTED;
    CUresult r;
    if (slabs == 1) {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
        cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
        cuuint32_t estr[2] = {1, 1};
        r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[3] = {(cuuint64_t)BK, (cuuint64_t)rows, (cuuint64_t)(K / BK)};
        cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)BK * 2};
        cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, (cuuint32_t)slabs};
        cuuint32_t estr[3] = {1, 1, 1};
        r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return PLM_ERR_ALIGN;
    std::lock_guard<std::mutex> g(lock);
    e.ptr = ptr; e.rows = rows; e.K = K; e.ld = ld; e.box_rows = box_rows; e.slabs = slabs; e.map = *map; e.used = true;
    return PLM_OK;
}


// What the fused forms of the product kernels need beside the product itself.
//
// An RMSNorm between two products is split over them.  The product before it (EPI_RESIDUAL) adds
// its result to the fp32 residual stream `out` in place, writes xw = bf16(new row * norm weight) for
// the product after it, and for every token the sum of squares of the new values that this CTA
// wrote, one row of ss_out per CTA that wrote part of the row.  The product after it (SCALE) multiplies in xw and
// scales token t's results by r[t] = 1 / sqrt(sum of those partial sums / size + eps): the
// normalisation commutes with the product.  All sums run in a fixed order.
struct Fuse {
    const float* scale_parts;   // SCALE: [n_parts, ld_parts], column t for token t
    int n_parts, ld_parts;
    float inv_size, eps;
    const bf16* norm_w;         // EPI_RESIDUAL: [F]
    bf16* xw;                   // EPI_RESIDUAL: [T, ld_xw]
    long ld_xw;
    float* ss_out;              // EPI_RESIDUAL: [rows as the kernel says, its own row length]
};

}  // namespace plm_tc
