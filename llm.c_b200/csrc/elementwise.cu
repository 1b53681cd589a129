// Stand-alone element-wise and column-reduction kernels: tanh-GELU forward (used when the GELU
// output is recomputed in the backward pass), GELU backward in place, and the bias gradient
// (column sums of a [rows, OC] gradient).  In the normal training path GELU and its derivative
// run inside the GEMM epilogues (gemm.cu); these kernels serve the recompute / unfused modes.
//
// The bias gradient is deterministic: every CTA folds a strip of rows for 256 columns in a fixed
// order and writes one fp32 partial row; a second kernel folds the strips in strip order.
//
// Capability parity: llmc/gelu.cuh and matmul_backward_bias_kernel9 / reduce_add_sum_kernel of
// llmc/matmul.cuh in the reference.
#include "common.cuh"

namespace {

__global__ void gelu_fwd_kernel(bf16* __restrict__ out, const bf16* __restrict__ inp, long long npack) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npack) return;
    bf16x8 a = ld128cs(inp + i * 8), o;
    #pragma unroll
    for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(gelu_fast(__bfloat162float(a[e])));
    st128(out + i * 8, o);
}

__global__ void gelu_bwd_kernel(bf16* __restrict__ d_inout, const bf16* __restrict__ inp, long long npack) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npack) return;
    bf16x8 a = ld128cs(inp + i * 8), d = ld128(d_inout + i * 8), o;
    #pragma unroll
    for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(gelu_grad_fast(__bfloat162float(a[e])) * __bfloat162float(d[e]));
    st128(d_inout + i * 8, o);
}

__global__ void residual_add_kernel(bf16* __restrict__ out, const bf16* __restrict__ a, const bf16* __restrict__ b, long long npack) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npack) return;
    bf16x8 x = ld128cs(a + i * 8), y = ld128cs(b + i * 8), o;
    #pragma unroll
    for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(__bfloat162float(x[e]) + __bfloat162float(y[e]));
    st128(out + i * 8, o);
}

constexpr int BG_WARPS = 8;
// grid (ceil(OC/256), strips). partials[strip][OC]
__global__ void __launch_bounds__(BG_WARPS * 32)
bias_grad_kernel(float* __restrict__ partials, const bf16* __restrict__ dout, int rows, int OC, int rows_per_strip) {
    __shared__ float sh[BG_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 256 + lane * 8;
    const int r0 = blockIdx.y * rows_per_strip, r1 = min(rows, r0 + rows_per_strip);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < OC) {
        for (int r = r0 + warp; r < r1; r += BG_WARPS) {
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
        for (int w = 0; w < BG_WARPS; w++) s += sh[w][c];
        partials[(size_t)blockIdx.y * OC + blockIdx.x * 256 + c] = s;
    }
}

__global__ void bias_grad_fold_kernel(bf16* __restrict__ dbias, const float* __restrict__ partials, int strips, int OC, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= OC) return;
    float s = 0.f;
    for (int i = 0; i < strips; i++) s += partials[(size_t)i * OC + c];
    if (accumulate) s += __bfloat162float(dbias[c]);
    dbias[c] = __float2bfloat16_rn(s);
}

int bg_strips(int rows, int OC) {
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int colgroups = CEIL_DIV(OC, 256);
    int strips = CEIL_DIV(4 * sms, colgroups);
    if (strips > CEIL_DIV(rows, BG_WARPS)) strips = CEIL_DIV(rows, BG_WARPS);
    if (strips < 1) strips = 1;
    return strips;
}

}  // namespace

extern "C" int llmc_gelu_fwd(bf16* out, const bf16* inp, long long n, cudaStream_t stream) {
    if (n % 8) return -1;
    gelu_fwd_kernel<<<(unsigned)CEIL_DIV(n / 8, 256), 256, 0, stream>>>(out, inp, n / 8);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
extern "C" int llmc_gelu_bwd_inplace(bf16* d_inout, const bf16* inp, long long n, cudaStream_t stream) {
    if (n % 8) return -1;
    gelu_bwd_kernel<<<(unsigned)CEIL_DIV(n / 8, 256), 256, 0, stream>>>(d_inout, inp, n / 8);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
extern "C" int llmc_residual_add(bf16* out, const bf16* a, const bf16* b, long long n, cudaStream_t stream) {
    if (n % 8) return -1;
    residual_add_kernel<<<(unsigned)CEIL_DIV(n / 8, 256), 256, 0, stream>>>(out, a, b, n / 8);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
extern "C" long long llmc_bias_grad_scratch(int rows, int OC) { return (long long)bg_strips(rows, OC) * OC; }
// dbias[c] (+)= sum_r dout[r, c]; scratch: llmc_bias_grad_scratch floats
extern "C" int llmc_bias_grad(bf16* dbias, float* scratch, const bf16* dout, int rows, int OC, int accumulate, cudaStream_t stream) {
    if (OC % 8) return -1;
    const int strips = bg_strips(rows, OC);
    const int rps = CEIL_DIV(rows, strips);
    bias_grad_kernel<<<dim3(CEIL_DIV(OC, 256), strips), BG_WARPS * 32, 0, stream>>>(scratch, dout, rows, OC, rps);
    CUDA_CHECK(cudaGetLastError());
    bias_grad_fold_kernel<<<CEIL_DIV(OC, 128), 128, 0, stream>>>(dbias, scratch, strips, OC, accumulate);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
