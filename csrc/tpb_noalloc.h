// Allocation-free entry point (no counterpart in the reference, which has no native code).
//
// Who needs it: callers that are not allowed to reach cudaMalloc / cudaFree or an allocator
// built on them while they run — code executing inside someone else's memory budget (an
// inference server that hands each plug-in a fixed arena), inside a region where the CUDA
// allocator lock must not be taken (a signal-safe or real-time thread), or in a process
// whose device memory is fully pre-committed at start-up.  tpb_rmsnorm_bwd() needs a
// zeroed fp32 accumulator for the weight gradient that such a caller has nowhere to get
// from; this variant keeps that accumulator inside the library.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest normalised dimension the built-in scratch covers (fp32 accumulator = 32 KiB per GPU,
// held by every GPU that loads the library until the process exits).
#define TPB_NOALLOC_MAX_DIM 8192

// Same math as tpb_rmsnorm_bwd (tpb.h): dx = d/dx [rmsnorm(x) * w] (+ dres), and the weight
// gradient summed over rows, but written as bf16 into `dw_bf16` [dim] (overwritten, not
// accumulated).  Inputs and outputs are the caller's; nothing is allocated or freed.
//
//  * The fp32 accumulator is a file-scope device array.  The first call on a device looks up
//    its address (cudaGetSymbolAddress) for that device; make that first call outside any
//    stream capture.
//  * All calls on a device share the accumulator and it keeps what the previous call left, so
//    every call clears it first (on `stream`).  Two calls whose kernels can overlap on the GPU
//    (different streams, no ordering between them) race on it: serialise them.
//  * dim must be a multiple of 8 and at most TPB_NOALLOC_MAX_DIM.
//
// Returns 0, or a negative code that tpb_noalloc_strerror() turns into a message:
//   -2 bad dim (not a multiple of 8), -6 dim above TPB_NOALLOC_MAX_DIM,
//   -7 scratch symbol lookup failed, 1000 + cudaError_t launch failure.
int tpb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, void* dw_bf16, int rows, int dim, void* stream);

const char* tpb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
