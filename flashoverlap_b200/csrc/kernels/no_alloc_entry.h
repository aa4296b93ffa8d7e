/* fo_gemm_rmsnorm_noalloc: GEMM + RMSNorm on one GPU without any allocation.
 *
 * This entry point has no counterpart in the reference.
 *
 * Who it is for.  Some hosts of this library may not allocate device memory
 * at the moment they need the kernel: an inference server that handed all of
 * its memory to a pool at start-up and runs with the allocator locked, a
 * plug-in inside another runtime that owns the device heap, or a latency
 * critical loop where cudaMalloc/cudaFree are forbidden because they can
 * synchronise the whole device.  The regular path
 * (OverlapImpl.gemm_rmsnorm) needs scratch memory from its caller (the
 * un-normalised product) and from a heap the library allocates lazily (the
 * tile arrival counters).  This variant keeps both in one array that is part
 * of the library image, so that a call consists of a small memset and one
 * kernel launch and nothing else.
 *
 * What it computes.  out[M,N] = RMSNorm(A[M,K] * B[N,K]^T) * gamma, the same
 * fused kernel as OverlapImpl.gemm_rmsnorm with the 128x256 tile: fp32
 * accumulation, the product rounded to the 16-bit type, fp32 row statistics.
 * A, B, gamma and out are device pointers supplied by the caller, row-major,
 * 16-byte aligned; dtype 0 = float16, 1 = bfloat16.
 *
 * Limits.  The scratch array holds FO_NOALLOC_MAX_ELEMS (16 Mi) product
 * values plus the counters: 32 MiB + 16 KiB of device memory on every GPU that
 * loads the library, held until the process exits.  M * N must not exceed
 * FO_NOALLOC_MAX_ELEMS, M must be a multiple of 128 (at most 128 * 2048), N a
 * multiple of 256, K a multiple of 8, and all four pointers 16-byte aligned;
 * anything else is refused with an error message before any work is enqueued.
 * At most 64 devices per process (device index 0..63).
 *
 * First call.  The first call on each device looks up the device address of
 * the scratch array (cudaGetSymbolAddress) and raises the kernel's
 * shared-memory limit for both dtypes.  Make that first call with the device current and
 * outside of any stream capture; later calls on that device only enqueue work
 * on `stream`.
 *
 * Sharing.  All calls on a device use the same scratch array, and the array
 * keeps what the previous call left in it.  The counters are cleared at the
 * start of every call, on `stream`.  Two calls whose kernels can overlap on
 * the GPU (different streams without an ordering between them) race on the
 * array and give wrong results: order them.
 *
 * Returns 0 on success.  On failure returns a non-zero code and, when `err` is
 * not null, writes a message of at most err_len - 1 characters into it.
 * `status32` may be null; otherwise it must point to 32 bytes of zeroed device
 * memory that receives the kernel's failure record (see StatusWord) should one
 * of its bounded waits expire.
 */
#ifndef FLASHOVERLAP_NO_ALLOC_ENTRY_H_
#define FLASHOVERLAP_NO_ALLOC_ENTRY_H_

#include <stddef.h>

#define FO_NOALLOC_MAX_ELEMS (16ll * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int fo_gemm_rmsnorm_noalloc(const void* A, const void* B, const void* gamma, void* out, int M, int N, int K,
                            int dtype, float eps, void* stream, void* status32, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif

#endif /* FLASHOVERLAP_NO_ALLOC_ENTRY_H_ */
