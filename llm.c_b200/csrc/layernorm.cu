// LayerNorm forward, fused residual-add + LayerNorm forward, and LayerNorm backward for bf16
// activations with fp32 statistics.
//
// Forward: one warp per row, 128-bit loads; the second and third pass over the row hit L1.
// Backward: each CTA walks a contiguous strip of rows with one thread per 8-channel pack, so every thread keeps the
// dweight/dbias partial sums of "its" channels in registers across the strip and writes one fp32 partial row per CTA;
// a second tiny kernel folds the CTA partials in a fixed order and accumulates into the bf16 gradients.
// No float atomics anywhere: results are bit-reproducible.
//
// Capability parity: llmc/layernorm.cuh (layernorm_forward, fused_residual_forward5,
// layernorm_backward) of the reference.
#include "common.cuh"

namespace {

constexpr int LNB_MAX_THREADS = 256;  // threads of a backward CTA: one per 8-channel pack of a row, up to this many
constexpr int LNB_MAX_CTAS_PER_SM = 16;

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

// Backward.  A CTA owns a strip of rows; thread t owns the 8-channel packs t, t + blockDim, ... (MAXP of them) of EVERY
// row, so
//   * the weights of its channels are converted to fp32 once,
//   * its dweight / dbias (/ column-sum) partial sums stay in registers for the whole strip,
//   * every row element is loaded exactly once, 128 bits at a time.
// The two row statistics need the whole row: one combined shuffle tree for both values, one shared-memory exchange and
// ONE barrier per row (the exchange buffer is double buffered by row parity).  With CACHE the fp32 values of the first
// pass (dout, dout * w, xhat) stay in registers for the second pass, which is then 2 FMAs per element for dinp plus the
// accumulations.  Per-CTA partial sums go to partials[cta][3][C]; a second kernel folds them in a fixed order.
// No float atomics: results are bit-reproducible.
DEVINL float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
DEVINL float bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

template <bool ACCUM_DINP, int MAXP, bool COLSUM, bool CACHE>
__global__ void __launch_bounds__(LNB_MAX_THREADS)
ln_bwd_col_kernel(bf16* __restrict__ dinp, float* __restrict__ partials, const bf16* __restrict__ dout,
                  const bf16* __restrict__ inp, const bf16* __restrict__ weight,
                  const float* __restrict__ mean, const float* __restrict__ rstd, int N, int C, int rows_per_cta) {
    __shared__ float2 red[2][LNB_MAX_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5, nthr = blockDim.x;
    const int npack = C >> 3;
    const int row0 = blockIdx.x * rows_per_cta;
    const int row1 = min(N, row0 + rows_per_cta);
    const float inv_c = 1.0f / C;
    float wf[MAXP][8], dw[MAXP][8], db[MAXP][8], dc[COLSUM ? MAXP : 1][8];
    #pragma unroll
    for (int i = 0; i < MAXP; i++) {
        const int p = tid + nthr * i;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (p < npack) w = *reinterpret_cast<const uint4*>(weight + p * 8);
        const uint32_t wu[4] = {w.x, w.y, w.z, w.w};
        #pragma unroll
        for (int k = 0; k < 4; k++) { wf[i][2 * k] = bf16lo(wu[k]); wf[i][2 * k + 1] = bf16hi(wu[k]); }
        #pragma unroll
        for (int e = 0; e < 8; e++) { dw[i][e] = 0.f; db[i][e] = 0.f; if (COLSUM) dc[i][e] = 0.f; }
    }
    // The loads of row r + 1 are issued before the arithmetic of row r (CACHE variants: few packs per thread, so the second
    // set of registers is cheap): a CTA then keeps two rows in flight instead of exposing the load latency once per row.
    constexpr bool PREFETCH = CACHE;
    uint4 ndq[PREFETCH ? MAXP : 1], nxq[PREFETCH ? MAXP : 1], noq[PREFETCH ? MAXP : 1];
    float nrs = 0.f, nmean = 0.f;
    auto load_row = [&](int row, uint4* dq_, uint4* xq_, uint4* oq_, float& rs_, float& mean_) {
        const size_t rb = (size_t)row * C;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = tid + nthr * i;
            dq_[i] = make_uint4(0u, 0u, 0u, 0u); xq_[i] = dq_[i]; oq_[i] = dq_[i];
            if (p < npack) {
                dq_[i] = __ldcs(reinterpret_cast<const uint4*>(dout + rb + p * 8));
                xq_[i] = __ldcs(reinterpret_cast<const uint4*>(inp + rb + p * 8));
                if (ACCUM_DINP) oq_[i] = __ldcs(reinterpret_cast<const uint4*>(dinp + rb + p * 8));
            }
        }
        rs_ = rstd[row];
        mean_ = mean[row];
    };
    if (PREFETCH && row0 < row1) load_row(row0, ndq, nxq, noq, nrs, nmean);
    for (int row = row0; row < row1; row++) {
        const size_t rbase = (size_t)row * C;
        uint4 dq[MAXP], xq[MAXP], oq[MAXP];
        float rs, mean_row;
        if (PREFETCH) {
            #pragma unroll
            for (int i = 0; i < MAXP; i++) { dq[i] = ndq[i]; xq[i] = nxq[i]; oq[i] = noq[i]; }
            rs = nrs; mean_row = nmean;
            if (row + 1 < row1) load_row(row + 1, ndq, nxq, noq, nrs, nmean);
        } else {
            load_row(row, dq, xq, oq, rs, mean_row);
        }
        const float mrs = -mean_row * rs;                          // xhat = x * rs + mrs
        float dy[CACHE ? MAXP : 1][8], dn[CACHE ? MAXP : 1][8], nn[CACHE ? MAXP : 1][8];
        float s1 = 0.f, s2 = 0.f;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const uint32_t du[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w}, xu[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w};
            #pragma unroll
            for (int e = 0; e < 8; e++) {
                const float d_ = (e & 1) ? bf16hi(du[e >> 1]) : bf16lo(du[e >> 1]);
                const float x_ = (e & 1) ? bf16hi(xu[e >> 1]) : bf16lo(xu[e >> 1]);
                const float dn_ = d_ * wf[i][e];
                const float nn_ = fmaf(x_, rs, mrs);
                s1 += dn_; s2 = fmaf(dn_, nn_, s2);
                if (CACHE) { dy[i][e] = d_; dn[i][e] = dn_; nn[i][e] = nn_; }
            }
        }
        // both sums through one shuffle tree: after the first exchange even lanes carry s1, odd lanes s2
        {
            const bool odd = lane & 1;
            float keep = odd ? s2 : s1;
            const float send = odd ? s1 : s2;
            keep += __shfl_xor_sync(0xffffffffu, send, 1);
            #pragma unroll
            for (int o_ = 2; o_ < 32; o_ <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o_);
            float* rb = reinterpret_cast<float*>(&red[row & 1][warp]);
            if (lane < 2) rb[lane] = keep;
        }
        __syncthreads();
        float t1 = 0.f, t2 = 0.f;
        for (int w = 0; w < nwarps; w++) { const float2 v = red[row & 1][w]; t1 += v.x; t2 += v.y; }
        // dinp = rs * (dn - mean(dn) - xhat * mean(dn * xhat)) = dn * rs + (xhat * c2 + c1)
        const float c1 = -t1 * inv_c * rs, c2 = -t2 * inv_c * rs;
        #pragma unroll
        for (int i = 0; i < MAXP; i++) {
            const int p = tid + nthr * i;
            const uint32_t du[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w}, xu[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w};
            const uint32_t ou[4] = {oq[i].x, oq[i].y, oq[i].z, oq[i].w};
            uint32_t res[4];
            #pragma unroll
            for (int k = 0; k < 4; k++) {
                float v[2];
                #pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const int e = 2 * k + hh;
                    float d_, dn_, nn_;
                    if (CACHE) { d_ = dy[i][e]; dn_ = dn[i][e]; nn_ = nn[i][e]; }
                    else {
                        d_ = hh ? bf16hi(du[k]) : bf16lo(du[k]);
                        const float x_ = hh ? bf16hi(xu[k]) : bf16lo(xu[k]);
                        dn_ = d_ * wf[i][e];
                        nn_ = fmaf(x_, rs, mrs);
                    }
                    db[i][e] += d_;
                    dw[i][e] = fmaf(d_, nn_, dw[i][e]);
                    float r_ = fmaf(dn_, rs, fmaf(nn_, c2, c1));
                    if (ACCUM_DINP) r_ += hh ? bf16hi(ou[k]) : bf16lo(ou[k]);
                    v[hh] = r_;
                }
                res[k] = pack_bf16x2(v[0], v[1]);
                if (COLSUM) { dc[i][2 * k] += bf16lo(res[k]); dc[i][2 * k + 1] += bf16hi(res[k]); }   // what the consumer of dinp reads
            }
            if (p < npack) *reinterpret_cast<uint4*>(dinp + rbase + p * 8) = make_uint4(res[0], res[1], res[2], res[3]);
        }
    }
    float* part = partials + (size_t)blockIdx.x * 3 * C;
    #pragma unroll
    for (int i = 0; i < MAXP; i++) {
        const int p = tid + nthr * i;
        if (p < npack) {
            #pragma unroll
            for (int e = 0; e < 8; e += 4) {
                *reinterpret_cast<float4*>(part + p * 8 + e) = make_float4(dw[i][e], dw[i][e + 1], dw[i][e + 2], dw[i][e + 3]);
                *reinterpret_cast<float4*>(part + C + p * 8 + e) = make_float4(db[i][e], db[i][e + 1], db[i][e + 2], db[i][e + 3]);
                if (COLSUM) *reinterpret_cast<float4*>(part + 2 * C + p * 8 + e) = make_float4(dc[i][e], dc[i][e + 1], dc[i][e + 2], dc[i][e + 3]);
            }
        }
    }
}

// dweight[c] (+)= sum over CTAs of partials, likewise dbias and (optionally) the column sums of dinp.  A block covers 16
// channels (4 threads x 4 floats) with 64 slices of CTAs; slice y adds CTAs y, y + 64, ... in order and the slices are added
// in order: a fixed tree.  (The first version used 24 blocks of scalar loads for 10 MB of partials and took a quarter of
// the operator's time.)
constexpr int LNB_FOLD_SLICES = 64;
DEVINL void add4(float4& a, const float4& b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }

__global__ void __launch_bounds__(4 * LNB_FOLD_SLICES)
ln_bwd_fold_kernel(bf16* __restrict__ dweight, bf16* __restrict__ dbias, bf16* __restrict__ dcolsum,
                   const float* __restrict__ partials, int num_ctas, int C, int accumulate, int accumulate_col) {
    __shared__ float4 sh[3][LNB_FOLD_SLICES][4];
    const int x = threadIdx.x & 3, y = threadIdx.x >> 2;
    const int c = blockIdx.x * 16 + x * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a, cs = a;
    if (c < C) {
        #pragma unroll 4
        for (int i = y; i < num_ctas; i += LNB_FOLD_SLICES) {
            const float* p = partials + (size_t)i * 3 * C + c;
            add4(a, __ldcs(reinterpret_cast<const float4*>(p)));
            add4(b, __ldcs(reinterpret_cast<const float4*>(p + C)));
            if (dcolsum) add4(cs, __ldcs(reinterpret_cast<const float4*>(p + 2 * C)));
        }
    }
    sh[0][y][x] = a; sh[1][y][x] = b; sh[2][y][x] = cs;
    __syncthreads();
    if (y == 0 && c < C) {
        a = make_float4(0.f, 0.f, 0.f, 0.f); b = a; cs = a;
        for (int k = 0; k < LNB_FOLD_SLICES; k++) { add4(a, sh[0][k][x]); add4(b, sh[1][k][x]); add4(cs, sh[2][k][x]); }
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w}, cv[4] = {cs.x, cs.y, cs.z, cs.w};
        #pragma unroll
        for (int e = 0; e < 4; e++) {
            float va = av[e], vb = bv[e], vc = cv[e];
            if (accumulate) { va += __bfloat162float(dweight[c + e]); vb += __bfloat162float(dbias[c + e]); }
            dweight[c + e] = __float2bfloat16_rn(va);
            dbias[c + e] = __float2bfloat16_rn(vb);
            if (dcolsum) {
                if (accumulate_col) vc += __bfloat162float(dcolsum[c + e]);
                dcolsum[c + e] = __float2bfloat16_rn(vc);
            }
        }
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
    return (long long)(LNB_MAX_CTAS_PER_SM * sms) * 3 * C;
}

namespace {
struct LnbLaunch { int threads, ctas, rows_per_cta; };

template <bool ACC, int MAXP, bool COL>
int lnb_launch(bf16* dinp, float* scratch, const bf16* dout, const bf16* inp, const bf16* weight, const float* mean, const float* rstd,
               int N, int C, int threads, int* ctas_out, cudaStream_t stream) {
    static int occ_cache[LNB_MAX_THREADS / 32 + 1] = {0};
    int& occ = occ_cache[threads / 32];
    if (occ == 0) {
        CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, ln_bwd_col_kernel<ACC, MAXP, COL, (MAXP <= 2)>, threads, 0));
        if (occ < 1) occ = 1;
        if (occ > LNB_MAX_CTAS_PER_SM) occ = LNB_MAX_CTAS_PER_SM;
    }
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int ctas = occ * sms;
    int rows_per_cta = CEIL_DIV(N, ctas);
    ctas = CEIL_DIV(N, rows_per_cta);
    ln_bwd_col_kernel<ACC, MAXP, COL, (MAXP <= 2)><<<ctas, threads, 0, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, rows_per_cta);
    CUDA_CHECK(cudaGetLastError());
    *ctas_out = ctas;
    return 0;
}

template <int MAXP>
int lnb_dispatch(bool acc, bool col, bf16* dinp, float* scratch, const bf16* dout, const bf16* inp, const bf16* weight,
                 const float* mean, const float* rstd, int N, int C, int threads, int* ctas_out, cudaStream_t stream) {
    if (acc) return col ? lnb_launch<true, MAXP, true>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, ctas_out, stream)
                        : lnb_launch<true, MAXP, false>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, ctas_out, stream);
    return col ? lnb_launch<false, MAXP, true>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, ctas_out, stream)
               : lnb_launch<false, MAXP, false>(dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, ctas_out, stream);
}
}  // namespace

// dinp (+)= dLN ; dweight, dbias (+)= column sums.  `scratch` holds llmc_layernorm_bwd_scratch floats.
// If dcolsum is given it receives (+)= the column sums of the final dinp: when dinp is the residual-stream gradient, that
// is the bias gradient of the projection that wrote into the residual stream, obtained without another pass.  C <= 16384.
extern "C" int llmc_layernorm_bwd(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                                  const bf16* weight, const float* mean, const float* rstd, int N, int C,
                                  int accumulate_dinp, int accumulate_dwdb, bf16* dcolsum, int accumulate_dcol, cudaStream_t stream) {
    if (C % 8 || C > LNB_MAX_THREADS * 8 * 8) return -1;
    const int npack = C / 8;
    const int threads = npack <= LNB_MAX_THREADS ? CEIL_DIV(npack, 32) * 32 : LNB_MAX_THREADS;
    const int packs = CEIL_DIV(npack, threads);
    const bool acc = accumulate_dinp != 0, col = dcolsum != nullptr;
    int ctas = 0, rc;
    if (packs <= 1) rc = lnb_dispatch<1>(acc, col, dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, &ctas, stream);
    else if (packs <= 2) rc = lnb_dispatch<2>(acc, col, dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, &ctas, stream);
    else if (packs <= 4) rc = lnb_dispatch<4>(acc, col, dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, &ctas, stream);
    else rc = lnb_dispatch<8>(acc, col, dinp, scratch, dout, inp, weight, mean, rstd, N, C, threads, &ctas, stream);
    if (rc) return rc;
    ln_bwd_fold_kernel<<<CEIL_DIV(C, 16), 4 * LNB_FOLD_SLICES, 0, stream>>>(dweight, dbias, dcolsum, scratch, ctas, C, accumulate_dwdb, accumulate_dcol);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
