// Allocation-free entry point of liblme_cuda.so.
//
// This function has no counterpart in the reference project; it exists for hosts that may not allocate device
// memory when they call into this library: a plug-in loaded into a serving process whose memory manager reserved
// the whole device at start-up (a later cudaMalloc fails or fragments its arena), a control loop that cannot
// accept the device-wide synchronisation an allocation may imply, or a plain C program that links the library and
// owns no allocator at all.  Such a caller still provides every input and output buffer; only the kernel's
// intermediate workspace comes from the library.
#pragma once
#include "lme_api.h"
#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in workspace, in floats (6.94 MiB per GPU that loads the library, held until the process
// exits).  A call needs lme_rmsnorm_bwd_partial_rows(T) * H floats and that function never returns more than
// LME_RMSNORM_BWD_MAX_PARTIAL_ROWS (444, lme_api.h): every H <= 4096 fits for any T (T >= 444 with H = 4096 uses
// the array to the last float), a wider H only for correspondingly few rows (T * H <= 444 * 4096).
#define LME_STATIC_SCRATCH_FLOATS (LME_RMSNORM_BWD_MAX_PARTIAL_ROWS * 4096)

// Same computation and arguments as lme_rmsnorm_bwd() minus the caller-provided `dw_partial` scratch: the per-CTA
// partial sums of the weight gradient go to a fixed array inside the library.
//
//   * Returns LME_ERR_TOO_LARGE (nothing is launched) when the problem needs more than LME_STATIC_SCRATCH_FLOATS.
//   * Calls no cudaMalloc / cudaFree and no allocating library routine.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current) and caches it; make that first call during start-up, before any stream capture begins.  The cache
//     is filled without a lock: two threads making the first call on one device at the same time both look the
//     address up and both store the same value.
//   * All calls on a device share the one array and it keeps whatever the previous call left.  This kernel writes
//     every workspace element it later reads, so nothing has to be cleared between calls - but two calls whose
//     kernels overlap on the GPU (different streams, no ordering between them) race on the array.  Serialise them.
int lme_rmsnorm_bwd_static_scratch(const void* dy, const void* h, const void* w, const float* rstd,
                                   const void* dres, void* dx, float* dw, int dw_accumulate, int T, int H,
                                   void* stream);

#ifdef __cplusplus
}
#endif
