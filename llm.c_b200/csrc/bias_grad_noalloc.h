// Allocation-free bias gradient.  This entry point has no counterpart in the reference; it exists
// for callers of this library that are not allowed to allocate device memory.
//
// Who cannot allocate: code that runs while a CUDA stream is being captured into a graph (an
// allocation is illegal there), callers that run under a fixed memory budget where every byte of
// the device is already handed out (a failed cudaMalloc in the middle of a step would kill the
// run), and hosts such as plug-ins or real-time loops that must not take the driver's allocation
// lock.  The ordinary llmc_bias_grad() needs a float scratch buffer that its caller has to
// allocate; this variant carries its scratch inside the library image instead.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the library reserves: LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS floats (4 MiB) of
// device memory per GPU that loads the library, held until the process exits.
#define LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS (1 << 20)

// dbias[c] (+)= sum over r of dout[r, c]      (dout: rows x OC bf16 row-major, dbias: OC bf16)
//
// dout must be aligned to 16 bytes (the kernel reads it with 128-bit loads; with OC a multiple of 8 every row then is);
// a view that starts at an odd offset of a larger tensor does not qualify.
//
// Returns 0 on success.  Returns -1 (and prints the reason to stderr) before any launch if OC is not a multiple of 8,
// if rows or OC is not positive, if a pointer is null or dout is not aligned to 16 bytes, or if the problem needs
// more scratch than the fixed array holds:
// OC must not exceed LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS.  (Wider problems still run; fewer row strips
// are used so that strips * OC fits the array.)  CUDA errors are returned as their cudaError_t value.
//
// The first call on each device looks up the device address of the scratch array (no allocation,
// but a runtime query): make that first call outside any stream capture.
// All calls on a device share the one array.  Two calls whose kernels may overlap on the GPU
// (different streams without an ordering between them) race on it; order them.  The array keeps the
// previous call's partial sums between calls; every word that a call reads it has written first, so
// nothing needs clearing.
// The function calls no cudaMalloc / cudaFree and no library routine that allocates.
int llmc_bias_grad_noalloc(__nv_bfloat16* dbias, const __nv_bfloat16* dout, int rows, int OC, int accumulate,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
