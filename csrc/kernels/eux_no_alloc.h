/* An entry point that allocates nothing. It has no counterpart in the reference.
 *
 * Who needs it: code that must not call cudaMalloc / cudaFree (or anything that
 * calls them) at the moment it wants a GEMM -- a latency-critical RPC handler
 * running inside a serving loop, a plug-in that runs under a host framework's
 * memory accounting, a region where allocation would synchronise the device or
 * is simply forbidden by the embedding application. The ordinary entry point
 * (eux_gemm_launch) needs two small scratch arrays from its caller (per-panel
 * arrival counters and a completion counter); this variant keeps that scratch
 * in a static device array inside the library instead, so the caller passes
 * only its inputs and its output.
 *
 *   Y[M,N] (bf16) = X[M,K] (bf16, in this GPU's memory) * W, with W given as Wt[N,K] (K-major)
 *
 * Limits and rules:
 *   - M <= EUX_NOALLOC_GEMM_MAX_M (the static array has one counter per 128 rows);
 *     a larger M is refused with EUX_ERR_TOO_LARGE and nothing is launched.
 *     M % 128 == 0, N % 256 == 0, K % 64 == 0 as for the ordinary entry point.
 *   - X must already be local: streaming X from a peer needs a staging buffer of
 *     M*K elements, which is not "modest", so that mode stays with eux_gemm_launch.
 *   - The static array (EUX_NOALLOC_GEMM_SCRATCH_BYTES) exists once per GPU that loads
 *     the library, for the life of the process.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress) and raises the kernel's shared-memory limit; make that
 *     first call before any stream capture begins.
 *   - Every call uses the same array and finds there what the previous call left, so the
 *     entry point clears it on `stream` before the kernel. Two calls whose kernels can
 *     overlap on the GPU (different streams, no dependency) race on it: keep calls on
 *     one stream or order them with events.
 *   - No cudaMalloc, cudaFree, or allocating library routine is called.
 * Returns 0, a cudaError_t, or an EUX_ERR_* value (see eux_error_string).
 */
#ifndef EUX_NO_ALLOC_H_
#define EUX_NO_ALLOC_H_

#include "eux_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define EUX_NOALLOC_GEMM_MAX_M 131072
#define EUX_NOALLOC_GEMM_SCRATCH_BYTES ((EUX_NOALLOC_GEMM_MAX_M / 128 + 64) * 4)

EUX_API int eux_gemm_bf16_noalloc(const void* x, const void* w_t, void* y, int M, int N, int K, uint32_t* status,
                                  uint64_t wait_timeout_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EUX_NO_ALLOC_H_ */
