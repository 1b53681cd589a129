// LayerNorm forward, fused residual-add + LayerNorm forward, and LayerNorm backward for bf16
// activations with fp32 statistics.
//
// Forward: one warp per row, 128-bit loads; the second and third pass over the row hit L1.
// Backward: each CTA walks a contiguous strip of rows; every lane keeps the dweight/dbias partial
// sums of "its" channels in registers across the strip, the CTA folds its warps in a fixed order
// and writes one fp32 partial row per CTA; a second tiny kernel folds the CTA partials in CTA order
// and accumulates into the bf16 gradients.  No float atomics anywhere: results are bit-reproducible.
//
// Capability parity: llmc/layernorm.cuh (layernorm_forward, fused_residual_forward5,
// layernorm_backward) of the reference.
#include "common.cuh"

namespace {

// Backward: MAXP packs (of 8 channels) per lane are held in registers => 32*8*MAXP channels per "slab"
// (MAXP = 3 covers C <= 768 with fewer registers, MAXP = 4 everything else; rows wider than a slab go slab by slab).
constexpr int LNB_WARPS = 4;         // warps per CTA of the backward kernel
constexpr int LNB_CTAS_PER_SM = 4;

template <bool FUSED_RESIDUAL>
__global__ void __launch_bounds__(256)
ln_fwd_kernel(bf16* __restrict__ out, float* __restrict__ mean_out, float* __restrict__ rstd_out,
              bf16* __restrict__ residual_out, const bf16* __restrict__ inp1, const bf16* __restrict__ inp2,
              const bf16* __restrict__ weight, const bf16* __restrict__ bias, int N, int C) {
    const int warps_per_block = blockDim.x >> 5;
    const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (row >= N) return;
    const int lane = threadIdx.x & 31;
    const int npack = C >> 3;
    const bf16* x1 = inp1 + (size_t)row * C;
    const bf16* x2 = FUSED_RESIDUAL ? inp2 + (size_t)row * C : nullptr;
    bf16* res = FUSED_RESIDUAL ? residual_out + (size_t)row * C : nullptr;

    // pass 1: (residual add,) sum
    float sum = 0.f;
    for (int p = lane; p < npack; p += 32) {
        bf16x8 a = ld128cs(x1 + p * 8);
        if (FUSED_RESIDUAL) {
            bf16x8 b = ld128cs(x2 + p * 8);
            #pragma unroll
            for (int e = 0; e < 8; e++) a[e] = __float2bfloat16_rn(__bfloat162float(a[e]) + __bfloat162float(b[e]));
            st128(res + p * 8, a);
        }
        #pragma unroll
        for (int e = 0; e < 8; e++) sum += __bfloat162float(a[e]);
    }
    const float mean = warp_sum(sum) / C;
    // pass 2: variance around the mean (the row is in L1 by now)
    const bf16* x = FUSED_RESIDUAL ? res : x1;
    if (FUSED_RESIDUAL) __syncwarp();
    float var = 0.f;
    for (int p = lane; p < npack; p += 32) {
        bf16x8 a = ld128(x + p * 8);
        #pragma unroll
        for (int e = 0; e < 8; e++) { float d = __bfloat162float(a[e]) - mean; var += d * d; }
    }
    const float rstd = rsqrtf(warp_sum(var) / C + 1e-5f);
    // pass 3: normalise
    bf16* o = out + (size_t)row * C;
    for (int p = lane; p < npack; p += 32) {
        bf16x8 a = ld128(x + p * 8);
        bf16x8 w = ld128(weight + p * 8);
        bf16x8 b = ld128(bias + p * 8);
        bf16x8 r;
        #pragma unroll
        for (int e = 0; e < 8; e++) {
            float n = (__bfloat162float(a[e]) - mean) * rstd;
            r[e] = __float2bfloat16_rn(n * __bfloat162float(w[e]) + __bfloat162float(b[e]));
        }
        st128cs(o + p * 8, r);
    }
    if (lane == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
    }
}

// dinp (+)= LN'(dout); per-CTA fp32 partials of dweight/dbias -> partials[cta][2][C].
// Fast path for rows that fit one warp's registers (C <= 256 * MAXP): the next row's dout / inp / dinp packs are requested
// before the current row is reduced (two rows of loads in flight per warp); the dweight / dbias partial sums of a warp
// live in its own slab of shared memory (conflict-free float4 layout), which keeps the register count low enough for
// four CTAs per SM.
template <bool ACCUM_DINP, int MAXP, bool COLSUM>
__global__ void __launch_bounds__(LNB_WARPS * 32, LNB_CTAS_PER_SM)
ln_bwd_fast_kernel(bf16* __restrict__ dinp, float* __restrict__ partials, const bf16* __restrict__ dout,
                   const bf16* __restrict__ inp, const bf16* __restrict__ weight,
                   const float* __restrict__ mean, const float* __restrict__ rstd, int N, int C, int rows_per_cta) {
    constexpr int NARR = COLSUM ? 3 : 2;
    extern __shared__ float4 sh4[];     // [warp][NARR (dw, db, column sums of dinp)][MAXP][2 halves][32 lanes]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int row0 = blockIdx.x * rows_per_cta;
    const int row1 = min(N, row0 + rows_per_cta);
    const int npack = C >> 3;
    float4* wacc = sh4 + (size_t)warp * (NARR * MAXP * 2 * 32);
    #pragma unroll
    for (int k = 0; k < NARR * MAXP * 2; k++) wacc[k * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);

    bf16x8 cd[MAXP], cx[MAXP], co[MAXP];
    float cm = 0.f, crs = 0.f;
    auto fetch = [&](int r, bf16x8* d, bf16x8* a, bf16x8* o, float& m_, float& rs_) {
        const bf16* dy = dout + (size_t)r * C;
        const bf16* x = inp + (size_t)r * C;
        const bf16* dx = dinp + (size_t)r * C;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = lane + 32 * i;
            if (p < npack) {
                d[i] = ld128cs(dy + p * 8); a[i] = ld128cs(x + p * 8);
                if (ACCUM_DINP) o[i] = ld128cs(dx + p * 8);
            }
        }
        m_ = mean[r]; rs_ = rstd[r];
    };
    int row = row0 + warp;
    if (row < row1) fetch(row, cd, cx, co, cm, crs);
    for (; row < row1; row += nwarps) {
        bf16x8 nd[MAXP], nx[MAXP], no[MAXP];
        float nm = 0.f, nrs = 0.f;
        const int nrow = row + nwarps;
        if (nrow < row1) fetch(nrow, nd, nx, no, nm, nrs);
        const float m = cm, rs = crs;
        float s1 = 0.f, s2 = 0.f;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = lane + 32 * i;
            if (p < npack) {
                bf16x8 w = ld128(weight + p * 8);
                #pragma unroll
                for (int e = 0; e < 8; e++) {
                    float dn = __bfloat162float(cd[i][e]) * __bfloat162float(w[e]);
                    float nn = (__bfloat162float(cx[i][e]) - m) * rs;
                    s1 += dn; s2 += dn * nn;
                }
            }
        }
        s1 = warp_sum(s1) / C; s2 = warp_sum(s2) / C;
        bf16* dx = dinp + (size_t)row * C;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = lane + 32 * i;
            if (p < npack) {
                bf16x8 w = ld128(weight + p * 8);
                bf16x8 o;
                float gw[8], gb[8], gc[8];
                #pragma unroll
                for (int e = 0; e < 8; e++) {
                    float dyv = __bfloat162float(cd[i][e]);
                    float nn = (__bfloat162float(cx[i][e]) - m) * rs;
                    float dn = dyv * __bfloat162float(w[e]);
                    gb[e] = dyv;
                    gw[e] = dyv * nn;
                    float v = (dn - s1 - nn * s2) * rs;
                    if (ACCUM_DINP) v += __bfloat162float(co[i][e]);
                    o[e] = __float2bfloat16_rn(v);
                    gc[e] = __bfloat162float(o[e]);      // what the consumer of dinp will read
                }
                st128(dx + p * 8, o);
                #pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    float4* aw = &wacc[((0 * MAXP + i) * 2 + hf) * 32 + lane];
                    float4* ab = &wacc[((1 * MAXP + i) * 2 + hf) * 32 + lane];
                    float4 tw = *aw, tb = *ab;
                    tw.x += gw[hf * 4 + 0]; tw.y += gw[hf * 4 + 1]; tw.z += gw[hf * 4 + 2]; tw.w += gw[hf * 4 + 3];
                    tb.x += gb[hf * 4 + 0]; tb.y += gb[hf * 4 + 1]; tb.z += gb[hf * 4 + 2]; tb.w += gb[hf * 4 + 3];
                    *aw = tw; *ab = tb;
                    if (COLSUM) {
                        float4* ac = &wacc[((2 * MAXP + i) * 2 + hf) * 32 + lane];
                        float4 tc = *ac;
                        tc.x += gc[hf * 4 + 0]; tc.y += gc[hf * 4 + 1]; tc.z += gc[hf * 4 + 2]; tc.w += gc[hf * 4 + 3];
                        *ac = tc;
                    }
                }
            }
        }
        #pragma unroll
        for (int i = 0; i < MAXP; i++) { cd[i] = nd[i]; cx[i] = nx[i]; co[i] = no[i]; }
        cm = nm; crs = nrs;
    }
    // fold the warps of this CTA in warp order
    __syncthreads();
    float* part = partials + (size_t)blockIdx.x * 3 * C;
    const float* shf = reinterpret_cast<const float*>(sh4);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const int p = c >> 3, e = c & 7;
        const int i = p >> 5, ln = p & 31, hf = e >> 2, comp = e & 3;
        float a = 0.f, b = 0.f, cs = 0.f;
        for (int w = 0; w < nwarps; w++) {
            const size_t base = (size_t)w * (NARR * MAXP * 2 * 32) * 4;
            a += shf[base + ((((0 * MAXP + i) * 2 + hf) * 32 + ln) * 4) + comp];
            b += shf[base + ((((1 * MAXP + i) * 2 + hf) * 32 + ln) * 4) + comp];
            if (COLSUM) cs += shf[base + ((((2 * MAXP + i) * 2 + hf) * 32 + ln) * 4) + comp];
        }
        part[c] = a;
        part[C + c] = b;
        if (COLSUM) part[2 * C + c] = cs;
    }
}

// Generic path (rows wider than one warp's registers): channel slabs of 1024, partial sums in registers.
template <bool ACCUM_DINP>
__global__ void __launch_bounds__(LNB_WARPS * 32)
ln_bwd_kernel(bf16* __restrict__ dinp, float* __restrict__ partials, const bf16* __restrict__ dout,
              const bf16* __restrict__ inp, const bf16* __restrict__ weight,
              const float* __restrict__ mean, const float* __restrict__ rstd, int N, int C, int rows_per_cta) {
    constexpr int MAXP = 4;
    extern __shared__ float sh[];   // [warps][2][slab] only during the fold
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int row0 = blockIdx.x * rows_per_cta;
    const int row1 = min(N, row0 + rows_per_cta);
    const int npack = C >> 3;
    const int slab_packs = 32 * MAXP;
    float* part = partials + (size_t)blockIdx.x * 3 * C;

    for (int slab0 = 0; slab0 < npack; slab0 += slab_packs) {
        float dw[MAXP][8], db[MAXP][8];
        #pragma unroll
        for (int i = 0; i < MAXP; i++)
            #pragma unroll
            for (int e = 0; e < 8; e++) { dw[i][e] = 0.f; db[i][e] = 0.f; }
        for (int row = row0 + warp; row < row1; row += nwarps) {
            const bf16* dy = dout + (size_t)row * C;
            const bf16* x = inp + (size_t)row * C;
            const float m = mean[row], rs = rstd[row];
            float s1 = 0.f, s2 = 0.f;           // row-wide sums (needed for every slab)
            for (int p = lane; p < npack; p += 32) {
                bf16x8 d = ld128(dy + p * 8), a = ld128(x + p * 8), w = ld128(weight + p * 8);
                #pragma unroll
                for (int e = 0; e < 8; e++) {
                    float dn = __bfloat162float(d[e]) * __bfloat162float(w[e]);
                    float nn = (__bfloat162float(a[e]) - m) * rs;
                    s1 += dn; s2 += dn * nn;
                }
            }
            s1 = warp_sum(s1) / C; s2 = warp_sum(s2) / C;
            bf16* dx = dinp + (size_t)row * C;
            #pragma unroll
            for (int i = 0; i < MAXP; i++) {
                const int p = slab0 + lane + 32 * i;
                if (p < npack) {
                    bf16x8 d = ld128(dy + p * 8), a = ld128(x + p * 8), w = ld128(weight + p * 8);
                    bf16x8 o;
                    if (ACCUM_DINP) o = ld128(dx + p * 8);
                    #pragma unroll
                    for (int e = 0; e < 8; e++) {
                        float dyv = __bfloat162float(d[e]);
                        float nn = (__bfloat162float(a[e]) - m) * rs;
                        float dn = dyv * __bfloat162float(w[e]);
                        db[i][e] += dyv;
                        dw[i][e] += dyv * nn;
                        float v = (dn - s1 - nn * s2) * rs;
                        if (ACCUM_DINP) v += __bfloat162float(o[e]);
                        o[e] = __float2bfloat16_rn(v);
                    }
                    st128(dx + p * 8, o);
                }
            }
        }
        // fold the warps of this CTA in warp order
        const int slab_ch = slab_packs * 8;
        __syncthreads();
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int lc = (lane + 32 * i) * 8;
            #pragma unroll
            for (int e = 0; e < 8; e++) {
                sh[(warp * 2 + 0) * slab_ch + lc + e] = dw[i][e];
                sh[(warp * 2 + 1) * slab_ch + lc + e] = db[i][e];
            }
        }
        __syncthreads();
        for (int c = threadIdx.x; c < slab_ch; c += blockDim.x) {
            const int gc = slab0 * 8 + c;
            if (gc < C) {
                float a = 0.f, b = 0.f;
                for (int w = 0; w < nwarps; w++) { a += sh[(w * 2 + 0) * slab_ch + c]; b += sh[(w * 2 + 1) * slab_ch + c]; }
                part[gc] = a;
                part[C + gc] = b;
            }
        }
        __syncthreads();
    }
}

// dweight[c] (+)= sum over CTAs (in CTA order) of partials; same for dbias and (optionally) the column sums of dinp
__global__ void ln_bwd_fold_kernel(bf16* __restrict__ dweight, bf16* __restrict__ dbias, bf16* __restrict__ dcolsum,
                                   const float* __restrict__ partials, int num_ctas, int C, int accumulate, int accumulate_col) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float a = 0.f, b = 0.f, cs = 0.f;
    for (int i = 0; i < num_ctas; i++) {
        a += partials[(size_t)i * 3 * C + c];
        b += partials[(size_t)i * 3 * C + C + c];
        if (dcolsum) cs += partials[(size_t)i * 3 * C + 2 * C + c];
    }
    if (accumulate) { a += __bfloat162float(dweight[c]); b += __bfloat162float(dbias[c]); }
    dweight[c] = __float2bfloat16_rn(a);
    dbias[c] = __float2bfloat16_rn(b);
    if (dcolsum) {
        if (accumulate_col) cs += __bfloat162float(dcolsum[c]);
        dcolsum[c] = __float2bfloat16_rn(cs);
    }
}

}  // namespace

extern "C" int llmc_layernorm_fwd(bf16* out, float* mean, float* rstd, const bf16* inp, const bf16* weight, const bf16* bias,
                                  int N, int C, cudaStream_t stream) {
    if (C % 8) return -1;
    ln_fwd_kernel<false><<<CEIL_DIV(N, 8), 256, 0, stream>>>(out, mean, rstd, nullptr, inp, nullptr, weight, bias, N, C);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// residual = inp1 + inp2 ; normed = LN(residual)
extern "C" int llmc_fused_residual_fwd(bf16* residual, bf16* normed, float* mean, float* rstd, const bf16* inp1, const bf16* inp2,
                                       const bf16* weight, const bf16* bias, int N, int C, cudaStream_t stream) {
    if (C % 8) return -1;
    ln_fwd_kernel<true><<<CEIL_DIV(N, 8), 256, 0, stream>>>(normed, mean, rstd, residual, inp1, inp2, weight, bias, N, C);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// Number of fp32 scratch elements llmc_layernorm_bwd needs
extern "C" long long llmc_layernorm_bwd_scratch(int N, int C) {
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    return (long long)(LNB_CTAS_PER_SM * sms) * 3 * C;
}

// dinp (+)= dLN ; dweight, dbias (+)= column sums.  `scratch` holds llmc_layernorm_bwd_scratch floats.
// If dcolsum is given (C <= 1024 only) it receives (+)= the column sums of the final dinp: when dinp is the residual-stream
// gradient, that is the bias gradient of the projection that wrote into the residual stream, obtained without another pass.
extern "C" int llmc_layernorm_bwd(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                                  const bf16* weight, const float* mean, const float* rstd, int N, int C,
                                  int accumulate_dinp, int accumulate_dwdb, bf16* dcolsum, int accumulate_dcol, cudaStream_t stream) {
    if (dcolsum != nullptr && C > 1024) return -2;
    if (C % 8) return -1;
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int ctas = LNB_CTAS_PER_SM * sms;
    int rows_per_cta = CEIL_DIV(N, ctas);
    ctas = CEIL_DIV(N, rows_per_cta);
    const int nwarps = LNB_WARPS;
    const size_t big = (size_t)nwarps * 3 * (32 * 4 * 8) * sizeof(float);      // 48 KB: the largest layout (3 arrays, 4 packs per lane)
    static bool configured = false;
    auto pick = [&](int maxp, bool acc, bool col) -> decltype(&ln_bwd_fast_kernel<true, 3, true>) {
        if (maxp == 3) return acc ? (col ? ln_bwd_fast_kernel<true, 3, true> : ln_bwd_fast_kernel<true, 3, false>)
                                  : (col ? ln_bwd_fast_kernel<false, 3, true> : ln_bwd_fast_kernel<false, 3, false>);
        return acc ? (col ? ln_bwd_fast_kernel<true, 4, true> : ln_bwd_fast_kernel<true, 4, false>)
                   : (col ? ln_bwd_fast_kernel<false, 4, true> : ln_bwd_fast_kernel<false, 4, false>);
    };
    if (!configured) {
        for (int mp = 3; mp <= 4; mp++)
            for (int acc = 0; acc < 2; acc++)
                for (int col = 0; col < 2; col++)
                    CUDA_CHECK(cudaFuncSetAttribute(pick(mp, acc, col), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big));
        CUDA_CHECK(cudaFuncSetAttribute(ln_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big));
        CUDA_CHECK(cudaFuncSetAttribute(ln_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big));
        configured = true;
    }
    if (C <= 1024) {
        const int maxp = (C <= 768) ? 3 : 4;
        const int narr = dcolsum ? 3 : 2;
        const size_t smem = (size_t)nwarps * narr * maxp * 2 * 32 * sizeof(float4);
        pick(maxp, accumulate_dinp != 0, dcolsum != nullptr)<<<ctas, nwarps * 32, smem, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, rows_per_cta);
    } else {
        auto kfn = accumulate_dinp ? ln_bwd_kernel<true> : ln_bwd_kernel<false>;
        kfn<<<ctas, nwarps * 32, (size_t)nwarps * 2 * (32 * 4 * 8) * sizeof(float), stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, rows_per_cta);
    }
    CUDA_CHECK(cudaGetLastError());
    ln_bwd_fold_kernel<<<CEIL_DIV(C, 128), 128, 0, stream>>>(dweight, dbias, dcolsum, scratch, ctas, C, accumulate_dwdb, accumulate_dcol);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
