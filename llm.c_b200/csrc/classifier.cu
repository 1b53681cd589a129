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
    constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
    // rows are processed back to front so that the rows the LM-head GEMM wrote last (still in L2) go first
    const int row = gridDim.x - 1 - blockIdx.x;
    bf16* x = logits + (size_t)row * Vp;
    if (threadIdx.x == 0) (void)LLMC_DBG_CHECK(targets[row] >= 0 && targets[row] < V, 0xC01);   // debug build: reported
    const int target = min(max(targets[row], 0), V - 1);       // ids are validated on the host; never index outside the row
    const int vpack = V >> 3;                 // full packs of valid columns
    // pass 1: running maximum and sum of 2^((x - max) * log2 e), per thread, one pack at a time
    float m = -INFINITY, s = 0.f;
    for (int p = threadIdx.x; p < vpack; p += CLS_THREADS) {
        bf16x8 a = ld128(x + p * 8);
        float f[8];
        float mx = m;
        #pragma unroll
        for (int e = 0; e < 8; e++) { f[e] = __bfloat162float(a[e]); mx = fmaxf(mx, f[e]); }
        const float off = mx * LOG2E;
        float add = 0.f;
        #pragma unroll
        for (int e = 0; e < 8; e++) add += ex2_fast(fmaf(f[e], LOG2E, -off));
        s = s * ex2_fast((m - mx) * LOG2E) + add;
        m = mx;
    }
    // ragged tail of valid columns (V not a multiple of 8)
    for (int c = vpack * 8 + threadIdx.x; c < V; c += CLS_THREADS) {
        float v = __bfloat162float(x[c]);
        float mx = fmaxf(m, v);
        s = s * ex2_fast((m - mx) * LOG2E) + ex2_fast((v - mx) * LOG2E);
        m = mx;
    }
    const float gmax = block_max(m, red);
    s = (m == -INFINITY) ? 0.f : s * ex2_fast((m - gmax) * LOG2E);
    const float gsum = block_sum(s, red);

    if (threadIdx.x == 0) {
        float lt = __bfloat162float(x[target]);
        float loss = -(lt - gmax - log2f(gsum) * LN2);
        if (accumulate_loss) losses[row] += loss; else losses[row] = loss;
    }
    if (!WRITE_DLOGITS) return;
    __syncthreads();    // the target logit has been read
    // pass 2 (the row is still in L2): dlogits = (softmax - onehot) * dloss; the vocabulary padding becomes zero
    const float goff = gmax * LOG2E;
    const float k = dloss / gsum;
    const int ppack = Vp >> 3;
    const int tpack = target >> 3;
    for (int p = threadIdx.x; p < ppack; p += CLS_THREADS) {
        bf16x8 a = ld128(x + p * 8);
        float g[8];
        #pragma unroll
        for (int e = 0; e < 8; e++) g[e] = ex2_fast(fmaf(__bfloat162float(a[e]), LOG2E, -goff)) * k;
        if (p == tpack) g[target & 7] -= dloss;
        if (p >= vpack) {                      // the pack that straddles V, and the padding
            #pragma unroll
            for (int e = 0; e < 8; e++) if (p * 8 + e >= V) g[e] = 0.f;
        }
        uint4 o;
        o.x = pack_bf16x2(g[0], g[1]); o.y = pack_bf16x2(g[2], g[3]); o.z = pack_bf16x2(g[4], g[5]); o.w = pack_bf16x2(g[6], g[7]);
        __stcs(reinterpret_cast<uint4*>(x + p * 8), o);
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
