// RMSNorm backward for callers that must not allocate.  This entry point has no counterpart in the
// reference project; it exists for users of this library only.
//
// Who needs it: code that runs where device-memory allocation is off limits — a latency-critical loop that
// may not take the allocator's locks or synchronisations, a plug-in running inside another framework's
// memory pool whose allocator must not be re-entered, or a process whose device-memory budget was fixed
// up front and may not grow.  The regular
// entry point (`vlmt_rmsnorm_bwd`, elementwise.h) asks its caller for a scratch tensor of per-block
// partial weight gradients, which in practice means an allocation per call.  This variant keeps that
// scratch in a fixed array that is part of the loaded library image, so it calls no cudaMalloc / cudaFree
// and no allocating library routine.
//
// Contract
//   * dy, x, dx: bf16 [rows, D]; w: bf16 (or fp32 when w_fp32 != 0) [D]; rstd: fp32 [rows];
//     dres: optional bf16 [rows, D] added to dx (may be null); dw: fp32 [D] OUTPUT (overwritten; with
//     rows <= 0 it is overwritten with zeros).
//   * D must be a multiple of 8 and at most VLMT_NOALLOC_MAX_D (8192).  Larger D is refused:
//     the function prints the reason to stderr and returns VLMT_NOALLOC_ERR_SIZE; nothing is launched.
//   * The scratch is VLMT_NOALLOC_MAX_BLOCKS x VLMT_NOALLOC_MAX_D floats (148 x 8192 x 4 B = 4.6 MiB).
//     Every GPU that loads the library holds it until the process exits, whether or not this function is
//     ever called.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current) and caches it.  Make that first call outside of any stream capture; later calls on
//     the same device do no set-up work.
//   * All calls on a device share the one array and it keeps whatever the previous call left in it.  The
//     kernels overwrite every slot they later read, so nothing has to be cleared between calls — but two
//     calls that overlap on the GPU (different streams, no ordering between them) race on it.  Order them.
//   * Returns 0, VLMT_NOALLOC_ERR_SIZE, VLMT_NOALLOC_ERR_SYMBOL (address lookup failed) or a positive
//     cudaError_t from the launches.
#pragma once
#include <cuda_runtime.h>

#define VLMT_NOALLOC_MAX_D 8192
#define VLMT_NOALLOC_MAX_BLOCKS 148
#define VLMT_NOALLOC_ERR_SIZE (-1)
#define VLMT_NOALLOC_ERR_SYMBOL (-2)

#ifdef __cplusplus
extern "C" {
#endif
int vlmt_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, int w_fp32, const float* rstd, const void* dres, void* dx,
                            float* dw, int rows, int D, int offset, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
