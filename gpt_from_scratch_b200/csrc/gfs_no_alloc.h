/* Split-K bf16 GEMM for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference implementation.
 *
 * Who needs it: code that runs where cudaMalloc / cudaFree are off limits - a host
 * thread inside a latency-critical serving loop that may not take the allocator's
 * device-wide synchronisation, a plugin loaded into a process whose memory budget is
 * fixed up front, or a caller that owns no allocator at all (plain C, another language
 * runtime) and can only hand over its own input and output buffers. The regular
 * gfs_gemm_bf16() needs the caller to supply an fp32 workspace for its split-K partial
 * tiles; such callers have nowhere to get one from.
 *
 * What it does instead: the partial tiles go to a fixed array that lives inside the
 * library image on the device (GFS_NO_ALLOC_SCRATCH_BYTES, reserved on every GPU that
 * loads the library until the process exits). The call performs no cudaMalloc, no
 * cudaFree and calls no allocating library routine; the tensor maps it needs are
 * encoded into variables on the host stack.
 *
 * Limits and rules:
 *  - splits * M * N * 4 bytes must fit in GFS_NO_ALLOC_SCRATCH_BYTES, otherwise the call
 *    is rejected with GFS_NO_ALLOC_ERR_TOO_LARGE and a message on stderr.
 *  - The first call on each device looks up the device address of the array
 *    (cudaGetSymbolAddress). Make that first call before starting any stream capture.
 *  - All calls share the one array. It keeps whatever the previous call left in it; that
 *    is harmless here because every partial element is written before it is read, so
 *    nothing has to start at zero. Two calls whose kernels overlap on the GPU (different
 *    streams, no dependency between them) race on the array: serialise them.
 *  - Waits inside the kernel are bounded as everywhere in this library, but this entry
 *    point does not report a timed-out wait (it has no status buffer to write to).
 */
#ifndef GFS_NO_ALLOC_H_
#define GFS_NO_ALLOC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GFS_NO_ALLOC_SCRATCH_BYTES (16u << 20) /* 16 MiB of fp32 partial tiles */

#define GFS_NO_ALLOC_ERR_BAD_ARGUMENT (-1)
#define GFS_NO_ALLOC_ERR_ALIGNMENT (-2)
#define GFS_NO_ALLOC_ERR_TENSOR_MAP (-3)
#define GFS_NO_ALLOC_ERR_TOO_LARGE (-4)
#define GFS_NO_ALLOC_ERR_SETUP (-5)
#define GFS_NO_ALLOC_ERR_LAUNCH (-6)

/* C[M,N] = op(A) op(B) (+ R when add != 0), bf16 in/out, fp32 accumulation, computed as
 * `splits` partial products over the contraction dimension that are summed in split order
 * (bitwise identical to gfs_gemm_bf16 with the same number of splits).
 * Operand layouts as for gfs_gemm_bf16: A is [M,K] (or [K,M] when a_mn_major), B is [N,K]
 * (or [K,N] when b_mn_major), row-major with leading dimensions in elements; all pointers
 * 16-byte aligned, N and the leading dimensions multiples of 8. splits >= 2 and at most
 * ceil(K/64). Returns 0 or one of the GFS_NO_ALLOC_ERR_* codes. */
int gfs_gemm_bf16_splitk_static(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda,
                                int ldb, int ldc, int ldr, int a_mn_major, int b_mn_major, int add, int splits,
                                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GFS_NO_ALLOC_H_ */
