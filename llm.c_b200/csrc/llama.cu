// Operators of the LLaMA-3 family that GPT-2 does not have: RMSNorm (forward, fused residual-add forward, backward),
// rotary position embedding fused with the grouped-query head expansion (forward and backward), and SwiGLU
// (forward and backward).  All are memory-bound passes over bf16 activations with fp32 math, 128-bit accesses and
// no float atomics (bit-reproducible results).
//
// Capability parity: the reference has these only as PyTorch modules (train_llama3.py: RMSNorm :133-146,
// apply_rotary_emb :107-117, repeat_kv :59-68, MLP :205-226); there is no CUDA counterpart to compare against.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------------------
// RMSNorm:  y = x * rsqrt(mean(x^2) + eps) * w            (statistics in fp32, one warp per row)

template <bool FUSED_RESIDUAL>
__global__ void __launch_bounds__(256)
rms_fwd_kernel(bf16* __restrict__ out, float* __restrict__ rstd_out, bf16* __restrict__ residual_out,
               const bf16* __restrict__ inp1, const bf16* __restrict__ inp2, const bf16* __restrict__ weight,
               int N, int C, float eps) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const int lane = threadIdx.x & 31;
    const int npack = C >> 3;
    const bf16* x1 = inp1 + (size_t)row * C;
    const bf16* x2 = FUSED_RESIDUAL ? inp2 + (size_t)row * C : nullptr;
    bf16* res = FUSED_RESIDUAL ? residual_out + (size_t)row * C : nullptr;
    float ss = 0.f;
    for (int p = lane; p < npack; p += 32) {
        bf16x8 a = ld128cs(x1 + p * 8);
        if (FUSED_RESIDUAL) {
            bf16x8 b = ld128cs(x2 + p * 8);
            #pragma unroll
            for (int e = 0; e < 8; e++) a[e] = __float2bfloat16_rn(__bfloat162float(a[e]) + __bfloat162float(b[e]));
            st128(res + p * 8, a);
        }
        #pragma unroll
        for (int e = 0; e < 8; e++) { float v = __bfloat162float(a[e]); ss += v * v; }
    }
    const float rstd = rsqrtf(warp_sum(ss) / C + eps);
    const bf16* x = FUSED_RESIDUAL ? res : x1;
    if (FUSED_RESIDUAL) __syncwarp();
    bf16* o = out + (size_t)row * C;
    for (int p = lane; p < npack; p += 32) {      // the row is in L1 by now
        bf16x8 a = ld128(x + p * 8);
        bf16x8 w = ld128(weight + p * 8);
        bf16x8 r;
        #pragma unroll
        for (int e = 0; e < 8; e++) {
            // the normalised value is rounded to the activation type before the weight is applied, as in the
            // reference module (`_norm(x.float()).type_as(x) * weight`)
            float n = __bfloat162float(__float2bfloat16_rn(__bfloat162float(a[e]) * rstd));
            r[e] = __float2bfloat16_rn(n * __bfloat162float(w[e]));
        }
        st128cs(o + p * 8, r);
    }
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
}

// Backward.  A CTA of RMSB_THREADS threads walks a strip of rows; thread t owns packs t, t + RMSB_THREADS, ... of every
// row (MAXP of them), so its dweight partial sums stay in registers over the whole strip and each row is read exactly
// once.  dinp (+)= rstd * (dn - xhat * mean(dn * xhat)) with dn = dout * w, xhat = x * rstd.
constexpr int RMSB_THREADS = 256;
constexpr int RMSB_CTAS_PER_SM = 4;

template <bool ACCUM_DINP, int MAXP>
__global__ void __launch_bounds__(RMSB_THREADS)
rms_bwd_kernel(bf16* __restrict__ dinp, float* __restrict__ partials, const bf16* __restrict__ dout,
               const bf16* __restrict__ inp, const bf16* __restrict__ weight, const float* __restrict__ rstd,
               int N, int C, int rows_per_cta) {
    __shared__ float red[2][RMSB_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int npack = C >> 3;
    const int row0 = blockIdx.x * rows_per_cta;
    const int row1 = min(N, row0 + rows_per_cta);
    float dw[MAXP][8];
    bf16x8 w[MAXP];
    #pragma unroll
    for (int i = 0; i < MAXP; i++) {
        const int p = tid + RMSB_THREADS * i;
        if (p < npack) w[i] = ld128(weight + p * 8);
        #pragma unroll
        for (int e = 0; e < 8; e++) dw[i][e] = 0.f;
    }
    for (int row = row0; row < row1; row++) {
        const bf16* dy = dout + (size_t)row * C;
        const bf16* x = inp + (size_t)row * C;
        bf16* dx = dinp + (size_t)row * C;
        const float rs = rstd[row];
        bf16x8 d[MAXP], a[MAXP], o[MAXP];
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = tid + RMSB_THREADS * i;
            if (p < npack) {
                d[i] = ld128cs(dy + p * 8); a[i] = ld128cs(x + p * 8);
                if (ACCUM_DINP) o[i] = ld128cs(dx + p * 8);
            }
        }
        float s = 0.f;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = tid + RMSB_THREADS * i;
            if (p < npack) {
                #pragma unroll
                for (int e = 0; e < 8; e++)
                    s += __bfloat162float(d[i][e]) * __bfloat162float(w[i][e]) * (__bfloat162float(a[i][e]) * rs);
            }
        }
        // block-wide sum, double buffered by row parity so one barrier per row is enough
        s = warp_sum(s);
        float* rb = red[row & 1];
        if (lane == 0) rb[warp] = s;
        __syncthreads();
        float tot = 0.f;
        #pragma unroll
        for (int k = 0; k < RMSB_THREADS / 32; k++) tot += rb[k];
        const float s2 = tot / C;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = tid + RMSB_THREADS * i;
            if (p < npack) {
                bf16x8 r;
                #pragma unroll
                for (int e = 0; e < 8; e++) {
                    float dyv = __bfloat162float(d[i][e]);
                    float nn = __bfloat162float(a[i][e]) * rs;
                    float dn = dyv * __bfloat162float(w[i][e]);
                    dw[i][e] += dyv * nn;
                    float v = (dn - nn * s2) * rs;
                    if (ACCUM_DINP) v += __bfloat162float(o[i][e]);
                    r[e] = __float2bfloat16_rn(v);
                }
                st128(dx + p * 8, r);
            }
        }
    }
    float* part = partials + (size_t)blockIdx.x * C;
    #pragma unroll
    for (int i = 0; i < MAXP; i++) {
        const int p = tid + RMSB_THREADS * i;
        if (p < npack) {
            #pragma unroll
            for (int e = 0; e < 8; e += 4)
                *reinterpret_cast<float4*>(part + p * 8 + e) = make_float4(dw[i][e], dw[i][e + 1], dw[i][e + 2], dw[i][e + 3]);
        }
    }
}

// dweight[c] (+)= sum over CTAs of the partial sums: a block covers 16 channels (4 threads x 4 floats) with 64 slices of CTAs;
// slice y adds CTAs y, y + 64, ... in order and the slices are added in order (a fixed tree, many loads in flight)
constexpr int RMS_FOLD_SLICES = 64;
__global__ void __launch_bounds__(4 * RMS_FOLD_SLICES)
rms_bwd_fold_kernel(bf16* __restrict__ dweight, const float* __restrict__ partials, int num_ctas, int C, int accumulate) {
    __shared__ float4 sh[RMS_FOLD_SLICES][4];
    const int x = threadIdx.x & 3, y = threadIdx.x >> 2;
    const int c = blockIdx.x * 16 + x * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < C) {
        #pragma unroll 4
        for (int i = y; i < num_ctas; i += RMS_FOLD_SLICES) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(partials + (size_t)i * C + c));
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
    }
    sh[y][x] = a;
    __syncthreads();
    if (y == 0 && c < C) {
        a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < RMS_FOLD_SLICES; k++) { const float4 v = sh[k][x]; a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
        const float av[4] = {a.x, a.y, a.z, a.w};
        #pragma unroll
        for (int e = 0; e < 4; e++) {
            float va = av[e];
            if (accumulate) va += __bfloat162float(dweight[c + e]);
            dweight[c + e] = __float2bfloat16_rn(va);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Rotary embedding + grouped-query expansion.
//   raw    (N, (NH + 2 NKV) * HS)   output of the QKV projection: NH query heads, NKV key heads, NKV value heads
//   packed (N, 3, NH, HS)           what the attention kernels read: every key / value head repeated NH / NKV times
// Adjacent element pairs (2j, 2j+1) of a query or key head are rotated by the angle t * freq_j; `freqs` holds
// (cos, sin) per (position, j).  One thread handles one 8-element pack (4 pairs).

DEVINL bf16x8 rotate_pack(const bf16x8& a, const float4& cs0, const float4& cs1, float sign) {
    bf16x8 r;
    const float c[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
    const float s[4] = {cs0.y * sign, cs0.w * sign, cs1.y * sign, cs1.w * sign};
    #pragma unroll
    for (int j = 0; j < 4; j++) {
        const float re = __bfloat162float(a[2 * j]), im = __bfloat162float(a[2 * j + 1]);
        r[2 * j] = __float2bfloat16_rn(re * c[j] - im * s[j]);
        r[2 * j + 1] = __float2bfloat16_rn(re * s[j] + im * c[j]);
    }
    return r;
}

__global__ void __launch_bounds__(256)
rope_fwd_kernel(bf16* __restrict__ packed, const bf16* __restrict__ raw, const float2* __restrict__ freqs,
                long long N, int T, int NH, int NKV, int HS) {
    const int hp = HS >> 3;
    const int heads = NH + 2 * NKV;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * heads * hp) return;
    const int p = (int)(idx % hp);
    const int h = (int)((idx / hp) % heads);
    const long long n = idx / ((long long)hp * heads);
    const int t = (int)(n % T);
    const int rep = NH / NKV;
    bf16x8 a = ld128cs(raw + (n * heads + h) * HS + p * 8);
    if (h < NH + NKV) {
        const float4* f = reinterpret_cast<const float4*>(freqs + (size_t)t * (HS >> 1) + p * 4);
        a = rotate_pack(a, f[0], f[1], 1.0f);
    }
    if (h < NH) {
        st128(packed + ((n * 3 + 0) * NH + h) * HS + p * 8, a);
    } else {
        const int which = (h < NH + NKV) ? 1 : 2;
        const int hk = (h - NH) - (which == 2 ? NKV : 0);
        for (int r = 0; r < rep; r++) st128(packed + ((n * 3 + which) * NH + hk * rep + r) * HS + p * 8, a);
    }
}

// draw = gradient of the projection output: queries and keys rotated back by the conjugate angle, the gradients of the
// repeated key / value heads summed over their group (fp32, fixed order) before the single rounding.
__global__ void __launch_bounds__(256)
rope_bwd_kernel(bf16* __restrict__ draw, const bf16* __restrict__ dpacked, const float2* __restrict__ freqs,
                long long N, int T, int NH, int NKV, int HS) {
    const int hp = HS >> 3;
    const int heads = NH + 2 * NKV;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * heads * hp) return;
    const int p = (int)(idx % hp);
    const int h = (int)((idx / hp) % heads);
    const long long n = idx / ((long long)hp * heads);
    const int t = (int)(n % T);
    const int rep = NH / NKV;
    bf16x8 a;
    if (h < NH) {
        a = ld128cs(dpacked + ((n * 3 + 0) * NH + h) * HS + p * 8);
    } else {
        const int which = (h < NH + NKV) ? 1 : 2;
        const int hk = (h - NH) - (which == 2 ? NKV : 0);
        float acc[8];
        #pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.f;
        for (int r = 0; r < rep; r++) {
            bf16x8 g = ld128cs(dpacked + ((n * 3 + which) * NH + hk * rep + r) * HS + p * 8);
            #pragma unroll
            for (int e = 0; e < 8; e++) acc[e] += __bfloat162float(g[e]);
        }
        if (which == 1) {
            // rotate the fp32 sum, round once
            const float4* f = reinterpret_cast<const float4*>(freqs + (size_t)t * (HS >> 1) + p * 4);
            const float4 cs0 = f[0], cs1 = f[1];
            const float c[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
            const float s[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
            #pragma unroll
            for (int j = 0; j < 4; j++) {
                const float re = acc[2 * j], im = acc[2 * j + 1];
                a[2 * j] = __float2bfloat16_rn(re * c[j] + im * s[j]);
                a[2 * j + 1] = __float2bfloat16_rn(im * c[j] - re * s[j]);
            }
        } else {
            #pragma unroll
            for (int e = 0; e < 8; e++) a[e] = __float2bfloat16_rn(acc[e]);
        }
        st128cs(draw + (n * heads + h) * HS + p * 8, a);
        return;
    }
    const float4* f = reinterpret_cast<const float4*>(freqs + (size_t)t * (HS >> 1) + p * 4);
    a = rotate_pack(a, f[0], f[1], -1.0f);
    st128cs(draw + (n * heads + h) * HS + p * 8, a);
}

// ---------------------------------------------------------------------------------------------------------------
// SwiGLU on the fused up-projection output x12 (N, 2H): x1 = x12[:, :H] (linear branch), x2 = x12[:, H:] (gate).
//   forward   h   = x1 * silu(x2)
//   backward  dx1 = dh * silu(x2) ;  dx2 = dh * x1 * sigmoid(x2) * (1 + x2 * (1 - sigmoid(x2)))

DEVINL float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(bf16* __restrict__ h, const bf16* __restrict__ x12, long long N, int H) {
    const int hp = H >> 3;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * hp) return;
    const int p = (int)(idx % hp);
    const long long n = idx / hp;
    const bf16* row = x12 + n * 2 * H;
    bf16x8 a = ld128cs(row + p * 8), g = ld128cs(row + H + p * 8), o;
    #pragma unroll
    for (int e = 0; e < 8; e++) {
        const float x2 = __bfloat162float(g[e]);
        o[e] = __float2bfloat16_rn(__bfloat162float(a[e]) * x2 * sigmoid_fast(x2));
    }
    st128cs(h + n * H + p * 8, o);
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(bf16* __restrict__ dx12, const bf16* __restrict__ dh, const bf16* __restrict__ x12, long long N, int H) {
    const int hp = H >> 3;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * hp) return;
    const int p = (int)(idx % hp);
    const long long n = idx / hp;
    const bf16* row = x12 + n * 2 * H;
    bf16x8 a = ld128cs(row + p * 8), g = ld128cs(row + H + p * 8), d = ld128cs(dh + n * H + p * 8), o1, o2;
    #pragma unroll
    for (int e = 0; e < 8; e++) {
        const float x1 = __bfloat162float(a[e]), x2 = __bfloat162float(g[e]), dy = __bfloat162float(d[e]);
        const float sg = sigmoid_fast(x2);
        o1[e] = __float2bfloat16_rn(dy * x2 * sg);
        o2[e] = __float2bfloat16_rn(dy * x1 * sg * (1.0f + x2 * (1.0f - sg)));
    }
    bf16* orow = dx12 + n * 2 * H;
    st128cs(orow + p * 8, o1);
    st128cs(orow + H + p * 8, o2);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// C entry points

extern "C" int llmc_rmsnorm_fwd(bf16* out, float* rstd, const bf16* inp, const bf16* weight, int N, int C, float eps, cudaStream_t stream) {
    if (C % 8) return -1;
    rms_fwd_kernel<false><<<CEIL_DIV(N, 8), 256, 0, stream>>>(out, rstd, nullptr, inp, nullptr, weight, N, C, eps);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// residual = inp1 + inp2 ; normed = RMSNorm(residual)
extern "C" int llmc_rmsnorm_fused_residual_fwd(bf16* residual, bf16* normed, float* rstd, const bf16* inp1, const bf16* inp2,
                                               const bf16* weight, int N, int C, float eps, cudaStream_t stream) {
    if (C % 8) return -1;
    rms_fwd_kernel<true><<<CEIL_DIV(N, 8), 256, 0, stream>>>(normed, rstd, residual, inp1, inp2, weight, N, C, eps);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" long long llmc_rmsnorm_bwd_scratch(int N, int C) {
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    return (long long)(RMSB_CTAS_PER_SM * sms) * C;
}

// dinp (+)= dRMSNorm(dout) ; dweight (+)= column sums of dout * xhat.  Rows up to 16384 channels.
extern "C" int llmc_rmsnorm_bwd(bf16* dinp, bf16* dweight, float* scratch, const bf16* dout, const bf16* inp, const bf16* weight,
                                const float* rstd, int N, int C, int accumulate_dinp, int accumulate_dw, cudaStream_t stream) {
    if (C % 8 || C > RMSB_THREADS * 8 * 8) return -1;
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int ctas = RMSB_CTAS_PER_SM * sms;
    int rows_per_cta = CEIL_DIV(N, ctas);
    ctas = CEIL_DIV(N, rows_per_cta);
    const int packs = CEIL_DIV(C / 8, RMSB_THREADS);
#define RMSB_LAUNCH(ACC, MP) rms_bwd_kernel<ACC, MP><<<ctas, RMSB_THREADS, 0, stream>>>(dinp, scratch, dout, inp, weight, rstd, N, C, rows_per_cta)
#define RMSB_PICK(MP) do { if (accumulate_dinp) RMSB_LAUNCH(true, MP); else RMSB_LAUNCH(false, MP); } while (0)
    if (packs <= 1) RMSB_PICK(1);
    else if (packs <= 2) RMSB_PICK(2);
    else if (packs <= 4) RMSB_PICK(4);
    else RMSB_PICK(8);
#undef RMSB_PICK
#undef RMSB_LAUNCH
    CUDA_CHECK(cudaGetLastError());
    rms_bwd_fold_kernel<<<CEIL_DIV(C, 16), 4 * RMS_FOLD_SLICES, 0, stream>>>(dweight, scratch, ctas, C, accumulate_dw);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

static int rope_check(int NH, int NKV, int HS) { return (HS % 8 || NKV <= 0 || NH % NKV) ? -1 : 0; }

extern "C" int llmc_rope_fwd(bf16* packed, const bf16* raw, const float* freqs, long long N, int T, int NH, int NKV, int HS, cudaStream_t stream) {
    if (rope_check(NH, NKV, HS)) return -1;
    const long long total = N * (NH + 2 * NKV) * (HS / 8);
    rope_fwd_kernel<<<(unsigned)CEIL_DIV(total, 256), 256, 0, stream>>>(packed, raw, reinterpret_cast<const float2*>(freqs), N, T, NH, NKV, HS);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_rope_bwd(bf16* draw, const bf16* dpacked, const float* freqs, long long N, int T, int NH, int NKV, int HS, cudaStream_t stream) {
    if (rope_check(NH, NKV, HS)) return -1;
    const long long total = N * (NH + 2 * NKV) * (HS / 8);
    rope_bwd_kernel<<<(unsigned)CEIL_DIV(total, 256), 256, 0, stream>>>(draw, dpacked, reinterpret_cast<const float2*>(freqs), N, T, NH, NKV, HS);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_swiglu_fwd(bf16* h, const bf16* x12, long long N, int H, cudaStream_t stream) {
    if (H % 8) return -1;
    swiglu_fwd_kernel<<<(unsigned)CEIL_DIV(N * (H / 8), 256), 256, 0, stream>>>(h, x12, N, H);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_swiglu_bwd(bf16* dx12, const bf16* dh, const bf16* x12, long long N, int H, cudaStream_t stream) {
    if (H % 8) return -1;
    swiglu_bwd_kernel<<<(unsigned)CEIL_DIV(N * (H / 8), 256), 256, 0, stream>>>(dx12, dh, x12, N, H);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
