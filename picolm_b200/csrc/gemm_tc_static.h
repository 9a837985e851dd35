/* picolm_b200: the skinny tensor-core matrix product without any allocation.
 *
 * This entry point has no counterpart in whoreson/picolm.  It exists for callers
 * that must not, or cannot, allocate device memory at the moment they need a
 * matrix product: a serving process that handed its whole device memory to a
 * planner of its own at start-up and has nothing left to ask cudaMalloc for; a
 * plug-in that runs inside another program's memory budget and is forbidden to
 * grow it; code on a latency path where a synchronising cudaMalloc or an
 * allocator's lock may not be taken.  Such callers bring their inputs and their
 * output; the fp32 partial sums that the split-K product needs in between live
 * in a fixed array inside the library instead of a buffer that somebody has to
 * allocate.
 *
 * The price: every GPU on which the library is loaded holds that array
 * (PLM_GEMM_TC_STATIC_SCRATCH_FLOATS floats, 16 MiB) from load to exit, problems
 * whose partial sums need more are refused, and all calls share the one array,
 * so two calls that overlap on the GPU (different streams, or one stream with
 * programmatic overlap) race on it.  Calls on one stream, one after another, are
 * safe, with one condition on `w`: the kernel requests its first tiles of `w`
 * before the kernel in front of it on the stream has finished (programmatic
 * dependent launch), so `w` must be complete before that kernel starts: weights
 * that were uploaded earlier are, the output of the product just before is not.
 * `x` and `out` have no such condition.
 */
#ifndef PICOLM_B200_GEMM_TC_STATIC_H
#define PICOLM_B200_GEMM_TC_STATIC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Floats of scratch that the library holds on every device. */
#define PLM_GEMM_TC_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

/* Refusals specific to this entry point (the other codes are those of plm_gemm_tc). */
#define PLM_ERR_SCRATCH_TOO_SMALL (-6)   /* the problem's partial sums exceed the fixed array */
#define PLM_ERR_SCRATCH_SETUP (-7)       /* the array's device address could not be obtained */

/* out[T, F] = x[T, K] * w[F, K]^T for T <= 64, bfloat16 operands, fp32 accumulation; out is
 * float32 (out_dtype 0) or bfloat16 (out_dtype 1) with leading dimension ldo.
 * Same arithmetic, same split of K and same result as plm_gemm_tc; only the
 * place of the partial sums differs.  `status` may be NULL; if given it is a
 * device int that stays 0 unless a bounded wait inside the kernel ran out.
 *
 * Calls cudaMalloc, cudaFree or any other allocating routine: never.
 *
 * The first call on a device looks up the array's device address (once per
 * device, with that device current).  Make that first call outside any stream
 * capture, e.g. with T = 0, which does the set-up and launches nothing.
 *
 * Nothing in the array has to start at zero: every partial sum is written
 * before it is read.  The array keeps the last call's partial sums afterwards.
 *
 * Returns 0 when the work was launched, a positive cudaError_t, or a negative
 * refusal; plm_gemm_tc_static_strerror turns a code into words. */
int plm_gemm_tc_static(const void* x, const void* w, void* out, int out_dtype, int T, int F, int K, long ldx,
                       long ldw, long ldo, int* status, cudaStream_t stream);

const char* plm_gemm_tc_static_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
