// Allocation-free entry point (this one has no counterpart in the reference project).
//
// Who needs it: hosts that drive these kernels from a context where the CUDA allocator
// must not be touched - a latency-critical serving or control loop that forbids
// cudaMalloc/cudaFree after start-up because they synchronise the device, a process
// whose memory budget was handed out in full at launch, or an embedding runtime that
// owns every allocation itself and only lends this library raw pointers.
//
// kmoe_rmsnorm_bwd_noalloc computes the same result as kmoe_rmsnorm_bwd (dx and the
// fp32 weight gradient of RMSNorm) but takes no scratch pointer: the per-row-slice
// partial sums live in a fixed array inside the library's device image
// (64 x KMOE_NOALLOC_MAX_D floats = 2 MiB, held by every GPU that loads the library
// until the process exits).  The caller still provides every input and output buffer.
//
// Rules of use:
//  * d must be a multiple of 8 and at most KMOE_NOALLOC_MAX_D; larger or misaligned
//    sizes are rejected with KMOE_NOALLOC_E_SIZE and nothing is launched.
//  * The first call on each device resolves the device address of the scratch array
//    (cudaGetSymbolAddress with that device current).  Make that first call during
//    set-up, before any stream capture begins.
//  * All calls on one device share the one scratch array.  The kernels overwrite the
//    part they use before reading it, so stale contents from an earlier call are never
//    read; but two calls that overlap in time on the same device (different streams)
//    race on it.  Serialise them.
//  * Host threads: the function may be entered from several host threads only if they
//    serialise their calls per device (which the shared scratch array demands anyway).  The
//    cached device address is written without a lock; concurrent first calls would store
//    the same value.
//  * The return code comes from cudaGetLastError after the launches, so an error left
//    pending by earlier unrelated work on the thread is reported as KMOE_NOALLOC_E_LAUNCH.
//  * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
#pragma once
#include <cuda_runtime.h>

#define KMOE_NOALLOC_MAX_D 8192
#define KMOE_NOALLOC_E_SIZE (-1)    /* d not a multiple of 8, d > KMOE_NOALLOC_MAX_D, or rows < 1 */
#define KMOE_NOALLOC_E_SYMBOL (-5)  /* the scratch symbol could not be resolved on this device */
#define KMOE_NOALLOC_E_LAUNCH (-2)  /* a kernel launch failed */

#ifdef __cplusplus
extern "C" {
#endif

// x, w, dy: bf16 (x, dy row-major [rows, d]; w [d]); rstd: fp32 [rows] as saved by the forward;
// dx: bf16 [rows, d] out; dw_f32: fp32 [d] out.  Returns 0 or one of the codes above.
int kmoe_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                             float* dw_f32, int rows, int d, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
