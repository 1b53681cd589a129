// Fused softmax + cross-entropy + dlogits over bf16 logits (N rows of Vp columns, the first V valid).
//
// One CTA per row.  Pass 1 computes the running maximum and the sum of exponentials (online
// softmax), pass 2 re-reads the row (it is still in L2: a row is ~100 KB) and overwrites it in place
// with (softmax - onehot(target)) * dloss.  HBM traffic is one read and one write of the logits.
// Columns V..Vp (vocabulary padding) are set to zero so the weight-gradient GEMM can consume the
// whole padded row.
//
// Capability parity: llmc/fused_classifier.cuh (fused_classifier) of the reference.
#include "common.cuh"

namespace {

constexpr int CLS_THREADS = 512;

template <bool WRITE_DLOGITS>
__global__ void __launch_bounds__(CLS_THREADS)
classifier_kernel(bf16* __restrict__ logits, float* __restrict__ losses, const int* __restrict__ targets,
                  float dloss, int V, int Vp, int accumulate_loss) {
    __shared__ float red[32];
    // rows are processed back to front so that the rows the LM-head GEMM wrote last (still in L2) go first
    const int row = gridDim.x - 1 - blockIdx.x;
    bf16* x = logits + (size_t)row * Vp;
    const int target = targets[row];
    const int vpack = V >> 3;                 // full packs of valid columns
    float m = -INFINITY, s = 0.f;
    for (int p = threadIdx.x; p < vpack; p += CLS_THREADS) {
        bf16x8 a = ld128(x + p * 8);
        float mx = m;
        #pragma unroll
        for (int e = 0; e < 8; e++) mx = fmaxf(mx, __bfloat162float(a[e]));
        float add = 0.f;
        #pragma unroll
        for (int e = 0; e < 8; e++) add += __expf(__bfloat162float(a[e]) - mx);
        s = s * __expf(m - mx) + add;
        m = mx;
    }
    // ragged tail of valid columns (V not a multiple of 8)
    for (int c = vpack * 8 + threadIdx.x; c < V; c += CLS_THREADS) {
        float v = __bfloat162float(x[c]);
        float mx = fmaxf(m, v);
        s = s * __expf(m - mx) + __expf(v - mx);
        m = mx;
    }
    const float gmax = block_max(m, red);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - gmax);
    const float gsum = block_sum(s, red);
    const float inv = 1.0f / gsum;

    if (threadIdx.x == 0) {
        float lt = __bfloat162float(x[target]);
        float loss = -(lt - gmax - logf(gsum));
        if (accumulate_loss) losses[row] += loss; else losses[row] = loss;
    }
    if (!WRITE_DLOGITS) return;
    __syncthreads();    // the target logit has been read
    const int ppack = Vp >> 3;
    for (int p = threadIdx.x; p < ppack; p += CLS_THREADS) {
        bf16x8 a = ld128(x + p * 8);
        bf16x8 o;
        #pragma unroll
        for (int e = 0; e < 8; e++) {
            const int c = p * 8 + e;
            float prob = __expf(__bfloat162float(a[e]) - gmax) * inv;
            float g = (prob - (c == target ? 1.0f : 0.0f)) * dloss;
            o[e] = (c < V) ? __float2bfloat16_rn(g) : __float2bfloat16_rn(0.f);
        }
        st128cs(x + p * 8, o);
    }
}

}  // namespace

// losses[row] (+)= -log softmax(logits[row])[target]; logits[row] <- dlogits (if write_dlogits)
extern "C" int llmc_fused_classifier(bf16* logits, float* losses, const int* targets, float dloss, int N, int V, int Vp,
                                     int write_dlogits, int accumulate_loss, cudaStream_t stream) {
    if (Vp % 8) return -1;
    if (write_dlogits) classifier_kernel<true><<<N, CLS_THREADS, 0, stream>>>(logits, losses, targets, dloss, V, Vp, accumulate_loss);
    else classifier_kernel<false><<<N, CLS_THREADS, 0, stream>>>(logits, losses, targets, dloss, V, Vp, accumulate_loss);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
