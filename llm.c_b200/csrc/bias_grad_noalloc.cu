// Bias gradient (column sums of a [rows, OC] bf16 gradient) that allocates nothing: the fp32 partial
// sums that the two-pass reduction needs live in a fixed array inside the library image.
// See bias_grad_noalloc.h for who needs this and for the contract.  No counterpart in the reference.
#include "bias_grad_noalloc.h"
#include "common.cuh"

// The scratch: strips x OC fp32 partial sums.  Being a file-scope __device__ array it is part of the
// module image: every GPU that loads the library holds these 4 MiB until the process ends.
static __device__ __align__(256) float g_noalloc_scratch[LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS];

namespace {

constexpr int NA_WARPS = 8;

// grid (ceil(OC/256), strips): each CTA sums its strip of rows for 256 columns, warps folded in warp order
__global__ void __launch_bounds__(NA_WARPS * 32)
na_bias_grad_partial_kernel(float* __restrict__ partials, const bf16* __restrict__ dout, int rows, int OC, int rows_per_strip) {
    __shared__ float sh[NA_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 256 + lane * 8;
    const int r0 = blockIdx.y * rows_per_strip, r1 = min(rows, r0 + rows_per_strip);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < OC) {
        for (int r = r0 + warp; r < r1; r += NA_WARPS) {
            bf16x8 d = ld128cs(dout + (size_t)r * OC + col);
            #pragma unroll
            for (int e = 0; e < 8; e++) acc[e] += __bfloat162float(d[e]);
        }
    }
    #pragma unroll
    for (int e = 0; e < 8; e++) sh[warp][lane * 8 + e] = acc[e];
    __syncthreads();
    const int c = threadIdx.x;
    if (blockIdx.x * 256 + c < OC) {
        float s = 0.f;
        #pragma unroll
        for (int w = 0; w < NA_WARPS; w++) s += sh[w][c];
        partials[(size_t)blockIdx.y * OC + blockIdx.x * 256 + c] = s;     // every (strip, column) word is written here
    }
}

// strips folded in strip order: the result does not depend on scheduling
__global__ void na_bias_grad_fold_kernel(bf16* __restrict__ dbias, const float* __restrict__ partials, int strips, int OC, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= OC) return;
    float s = 0.f;
    for (int i = 0; i < strips; i++) s += partials[(size_t)i * OC + c];
    if (accumulate) s += __bfloat162float(dbias[c]);
    dbias[c] = __float2bfloat16_rn(s);
}

// Device address of the scratch array, looked up once per device.  In host code the name
// g_noalloc_scratch is only a handle for the runtime, not an address a kernel could use, hence the query.
// The cache is filled without a lock: host threads that race on a device's first call all store the same
// address, so the worst case is a repeated query.
constexpr int NA_MAX_DEVICES = 64;
float* g_scratch_addr[NA_MAX_DEVICES] = {nullptr};

int scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NA_MAX_DEVICES) { fprintf(stderr, "[llmc_b200] bias_grad_noalloc: device index %d out of range\n", dev); return -1; }
    if (g_scratch_addr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);      // with device `dev` current
        if (e != cudaSuccess || p == nullptr) {
            fprintf(stderr, "[llmc_b200] bias_grad_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : -1;
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int llmc_bias_grad_noalloc(__nv_bfloat16* dbias, const __nv_bfloat16* dout, int rows, int OC, int accumulate,
                                      cudaStream_t stream) {
    if (rows <= 0 || OC <= 0 || (OC % 8) != 0) {
        fprintf(stderr, "[llmc_b200] bias_grad_noalloc: need rows > 0 and OC a positive multiple of 8 (got rows %d, OC %d)\n", rows, OC);
        return -1;
    }
    if (dbias == nullptr || dout == nullptr || (reinterpret_cast<uintptr_t>(dout) & 15u) != 0 || (reinterpret_cast<uintptr_t>(dbias) & 1u) != 0) {
        fprintf(stderr, "[llmc_b200] bias_grad_noalloc: dout must be a non-null pointer aligned to 16 bytes and dbias a non-null bf16 pointer\n");
        return -1;
    }
    if (OC > LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS) {
        fprintf(stderr, "[llmc_b200] bias_grad_noalloc: OC = %d exceeds the built-in scratch of %d floats; use llmc_bias_grad with a "
                        "caller-provided buffer\n", OC, LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS);
        return -1;
    }
    float* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int colgroups = CEIL_DIV(OC, 256);
    int strips = CEIL_DIV(4 * sms, colgroups);
    if (strips > CEIL_DIV(rows, NA_WARPS)) strips = CEIL_DIV(rows, NA_WARPS);
    const int fit = LLMC_BIAS_GRAD_NOALLOC_MAX_FLOATS / OC;       // >= 1 by the check above
    if (strips > fit) strips = fit;
    if (strips < 1) strips = 1;
    const int rows_per_strip = CEIL_DIV(rows, strips);
    strips = CEIL_DIV(rows, rows_per_strip);
    na_bias_grad_partial_kernel<<<dim3(colgroups, strips), NA_WARPS * 32, 0, stream>>>(scratch, dout, rows, OC, rows_per_strip);
    CUDA_CHECK(cudaGetLastError());
    na_bias_grad_fold_kernel<<<CEIL_DIV(OC, 128), 128, 0, stream>>>(dbias, scratch, strips, OC, accumulate);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
