// Shared device helpers of the picolm_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

// Tokens per cache page.  The cache, the step metadata and every kernel that
// walks a block table agree on this one number.
#define PLM_PAGE 64

// Return codes of the extern "C" entry points: 0 = launched, > 0 = a cudaError_t,
// < 0 = the arguments were refused before any launch.
#define PLM_OK 0
#define PLM_ERR_DTYPE (-1)
#define PLM_ERR_SHAPE (-2)
#define PLM_ERR_ALIGN (-3)
#define PLM_ERR_UNSUPPORTED (-4)

// SMs of a B200, the one target of these kernels (sm_100a): what grids, split factors and wave sizes are
// planned for.  A plan must not depend on the device it is made on (the same shapes must give the same
// order of sums everywhere), so this is a constant and not a device attribute; ops/_lib.py's SM_COUNT is
// the same number (tests/test_config.py compares the two).
#define PLM_SM_COUNT 148

// dtype codes shared with the Python side
#define PLM_F32 0
#define PLM_BF16 1

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NT threads (NT a multiple of 32, at most 1024); every
// thread gets the result.  `red` is shared scratch of at least 33 floats.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = (lane < NT / 32) ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// One rotary pair (picolm/tensor.c:3216-3304: x0' = x0 c - x1 s, x1' = x0 s + x1 c) with the roundings spelt
// out (each product rounded, then the sum: what a plain implementation does), so that every kernel that
// rotates gives the same bits whatever the compiler would fuse.
__device__ __forceinline__ float rope_first(float a, float b, float c, float s) { return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)); }
__device__ __forceinline__ float rope_second(float a, float b, float c, float s) { return __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)); }

// Programmatic dependent launch.  A kernel launched through launch_pdl may begin while the kernel
// before it on the stream is still running; pdl_wait() blocks until that kernel (and with it every
// earlier one) has finished and its writes are visible.  So: before pdl_wait() a kernel may only
// set itself up and read what no earlier kernel of the step writes (weights); it must not write
// global memory.  pdl_launch_dependents() lets the next kernel begin its own set-up.  Without the
// launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with a thread-block cluster of `cluster` CTAs (the grid must be a multiple of it in every
// dimension).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                             cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster.x;
    attr[1].val.clusterDim.y = cluster.y;
    attr[1].val.clusterDim.z = cluster.z;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Thread-block clusters: the rank of this CTA, a barrier over all threads of the cluster (its
// release/acquire pair makes shared-memory writes before it visible to reads after it), and loads
// from another CTA's shared memory (an address of this CTA's shared memory mapped to that rank).
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(const void* local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t cluster_map_addr(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// The checked build (-DPLM_CHECK; the serving build has none of this).  The kernels that follow indices
// which the host computed (page numbers from a page table, a token's sequence and position, gathered rows)
// compare every such index with its bound before they use it.  An index outside its bound is not followed:
// the status word gets the kind of index (16 page, 17 sequence, 18 position, 19 row; the first one wins),
// and index 0 is used in its place (page 0 is the cache's null page).  The bounds are set per library by
// plm_check_bounds, on the stream, before the launches they are meant for; a bound of 0 is not checked.
// This is what stands in for a memory checker where none can be run; the reference's counterparts are its
// address-sanitizer build and its attention stress test (picolm/Makefile:249-250, picolm/picolm.c:661-761).
#ifdef PLM_CHECK
struct PlmBounds {
    int n_pages, n_seqs, n_positions, n_rows;
    int* status;
};
__device__ PlmBounds plm_bounds = {0, 0, 0, 0, nullptr};
__device__ __forceinline__ int plm_checked(int v, int limit, int kind) {
    if (limit > 0 && (unsigned)v >= (unsigned)limit) {
        if (plm_bounds.status) atomicCAS(plm_bounds.status, 0, kind);
        return 0;
    }
    return v;
}
#define PLM_PAGE_NO(p) plm_checked((p), plm_bounds.n_pages, 16)
#define PLM_SEQ_NO(s) plm_checked((s), plm_bounds.n_seqs, 17)
#define PLM_POSITION(p) plm_checked((p), plm_bounds.n_positions, 18)
#define PLM_ROW_NO(r) plm_checked((r), plm_bounds.n_rows, 19)
extern "C" int plm_check_bounds(int n_pages, int n_seqs, int n_positions, int n_rows, int* status, cudaStream_t stream) {
    const PlmBounds b = {n_pages, n_seqs, n_positions, n_rows, status};
    cudaError_t e = cudaMemcpyToSymbolAsync(plm_bounds, &b, sizeof(b), 0, cudaMemcpyHostToDevice, stream);
    return e == cudaSuccess ? PLM_OK : (int)e;
}
#else
#define PLM_PAGE_NO(p) (p)
#define PLM_SEQ_NO(s) (s)
#define PLM_POSITION(p) (p)
#define PLM_ROW_NO(r) (r)
#endif

static inline int plm_status_of(cudaError_t e) { return e == cudaSuccess ? PLM_OK : (int)e; }

static inline int plm_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? PLM_OK : (int)e;
}
