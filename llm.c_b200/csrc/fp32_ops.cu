// Full-precision (fp32) kernels of the GPT-2 operator set: token + position embedding forward / backward, LayerNorm forward
// (optionally fused with the residual add) and backward, tanh-GELU forward / backward, residual add, bias gradient, fused
// softmax + cross-entropy classifier, causal softmax forward / backward and the head permutations of the attention block
// (whose two batched products run on the vendor library, as in the reference's legacy trainer), AdamW and the squared
// gradient norm.  Every tensor is float; 16-byte accesses move 4 elements.  All reductions have a fixed order: results are
// bit-reproducible from run to run.
//
// This is the device side of the trainer's "-dt fp32" mode (the matmuls of that mode are gemm_tf32.cu or cuBLAS in IEEE fp32).
// Capability parity: the kernels of train_gpt2_fp32.cu in the reference (encoder_forward_kernel3, layernorm_forward_kernel3,
// layernorm_backward_kernel2, softmax_forward_kernel5, softmax_autoregressive_backward_kernel, gelu_*_kernel,
// matmul_backward_bias_kernel4, fused_classifier_kernel3, adamw_kernel2, permute / unpermute kernels).
#include "common.cuh"

namespace {

using f32x4 = Pack128<float>;

DEVINL float gelu_exact_tanh(float x) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}
DEVINL float gelu_exact_tanh_grad(float x) {
    const float k = 0.7978845608028654f;
    const float x2 = x * x;
    const float t = tanhf(k * x * (1.0f + 0.044715f * x2));
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k * (1.0f + 3.0f * 0.044715f * x2);
}

// ---------------------------------------------------------------------------------------------------------------------
// element-wise

__global__ void gelu_fwd_f32(float* __restrict__ out, const float* __restrict__ inp, long long npack) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npack) return;
    f32x4 a = ld128cs(inp + i * 4), o;
    #pragma unroll
    for (int e = 0; e < 4; e++) o[e] = gelu_exact_tanh(a[e]);
    st128(out + i * 4, o);
}

__global__ void gelu_bwd_f32(float* __restrict__ d_inout, const float* __restrict__ inp, long long npack) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npack) return;
    f32x4 a = ld128cs(inp + i * 4), d = ld128(d_inout + i * 4), o;
    #pragma unroll
    for (int e = 0; e < 4; e++) o[e] = gelu_exact_tanh_grad(a[e]) * d[e];
    st128(d_inout + i * 4, o);
}

__global__ void residual_add_f32(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, long long npack) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npack) return;
    f32x4 x = ld128cs(a + i * 4), y = ld128cs(b + i * 4), o;
    #pragma unroll
    for (int e = 0; e < 4; e++) o[e] = x[e] + y[e];
    st128(out + i * 4, o);
}

// ---------------------------------------------------------------------------------------------------------------------
// embeddings

__global__ void encoder_fwd_f32(float* __restrict__ out, const int* __restrict__ tokens, const float* __restrict__ wte,
                                const float* __restrict__ wpe, int B, int T, int C, int V) {
    const int cp = C >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * T * cp) return;
    const int p = (int)(idx % cp);
    const long long bt = idx / cp;
    const int t = (int)(bt % T);
    (void)LLMC_DBG_CHECK(tokens[bt] >= 0 && tokens[bt] < V, 0xE01);     // debug build: an id outside the table is reported
    const int tok = min(max(tokens[bt], 0), V - 1);
    f32x4 o = ld128(wte + (size_t)tok * C + p * 4);
    if (wpe != nullptr) {
        const f32x4 b = ld128(wpe + (size_t)t * C + p * 4);
        #pragma unroll
        for (int e = 0; e < 4; e++) o[e] += b[e];
    }
    st128cs(out + bt * C + p * 4, o);
}

// dwpe[t, c] (+)= sum over b (ascending) of dout[b, t, c]
__global__ void wpe_bwd_f32(float* __restrict__ dwpe, const float* __restrict__ dout, int B, int T, int C, int accumulate) {
    const int cp = C >> 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * cp) return;
    const int p = idx % cp, t = idx / cp;
    f32x4 acc = f32x4::zeros();
    for (int b = 0; b < B; b++) {
        const f32x4 d = ld128cs(dout + ((size_t)b * T + t) * C + p * 4);
        #pragma unroll
        for (int e = 0; e < 4; e++) acc[e] += d[e];
    }
    float* dst = dwpe + (size_t)t * C + p * 4;
    if (accumulate) {
        const f32x4 old = ld128(dst);
        #pragma unroll
        for (int e = 0; e < 4; e++) acc[e] += old[e];
    }
    st128(dst, acc);
}

constexpr int IDS_PER_CTA = 64;
constexpr int LIST_CAP = 4096;
constexpr int WTE_THREADS = 256;
constexpr int WTE_MAXP = 8;          // float4 packs per lane and pass: 1024 channels per pass

// dwte[v, :] (+)= sum over the positions i (ascending) with tokens[i] == v of dout[i, :].  A CTA owns 64 consecutive ids: it
// scans the token array in position order, keeps the positions that hit its ids (sorted by construction), and each warp sums
// the rows of "its" ids in that order: one writer per table row, no atomics.
__global__ void __launch_bounds__(WTE_THREADS)
wte_bwd_f32(float* __restrict__ dwte, const float* __restrict__ dout, const int* __restrict__ tokens, int N, int C, int V, int accumulate) {
    __shared__ int list_pos[LIST_CAP];
    __shared__ unsigned char list_id[LIST_CAP];
    __shared__ int warp_counts[WTE_THREADS / 32];
    __shared__ int list_len;
    __shared__ int touched[IDS_PER_CTA];
    const int v0 = blockIdx.x * IDS_PER_CTA;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int nwarps = WTE_THREADS / 32;
    const int npack = C >> 2;
    if (threadIdx.x < IDS_PER_CTA) touched[threadIdx.x] = 0;
    if (threadIdx.x == 0) list_len = 0;
    __syncthreads();
    int pos0 = 0;
    while (pos0 < N) {
        while (pos0 < N) {
            if (list_len + WTE_THREADS > LIST_CAP) break;        // uniform: list_len is read after a barrier
            const int i = pos0 + threadIdx.x;
            const int tok = (i < N) ? tokens[i] : -1;
            const bool hit = (tok >= v0) && (tok < v0 + IDS_PER_CTA);
            const unsigned ballot = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) warp_counts[warp] = __popc(ballot);
            __syncthreads();
            int base = list_len;
            for (int w = 0; w < warp; w++) base += warp_counts[w];
            if (hit) {
                const int slot = base + __popc(ballot & ((1u << lane) - 1u));
                list_pos[slot] = i;
                list_id[slot] = (unsigned char)(tok - v0);
            }
            __syncthreads();
            if (threadIdx.x == 0) { int tot = 0; for (int w = 0; w < nwarps; w++) tot += warp_counts[w]; list_len += tot; }
            __syncthreads();
            pos0 += WTE_THREADS;
        }
        const int len = list_len;
        for (int id = warp; id < IDS_PER_CTA; id += nwarps) {
            const int v = v0 + id;
            if (v >= V) break;
            for (int pbase = 0; pbase < npack; pbase += 32 * WTE_MAXP) {
                f32x4 acc[WTE_MAXP];
                #pragma unroll
                for (int i = 0; i < WTE_MAXP; i++) acc[i] = f32x4::zeros();
                bool any = false;
                for (int l0 = 0; l0 < len; l0 += 32) {
                    const int l = l0 + lane;
                    const bool mine = (l < len) && (list_id[l] == id);
                    unsigned m = __ballot_sync(0xffffffffu, mine);
                    while (m) {
                        const int j = __ffs(m) - 1;
                        m &= m - 1;
                        any = true;
                        const float* src = dout + (size_t)list_pos[l0 + j] * C;
                        #pragma unroll
                        for (int i = 0; i < WTE_MAXP; i++) {
                            const int p = pbase + lane + 32 * i;
                            if (p < npack) {
                                const f32x4 d = ld128cs(src + p * 4);
                                #pragma unroll
                                for (int e = 0; e < 4; e++) acc[i][e] += d[e];
                            }
                        }
                    }
                }
                const bool add_old = accumulate || touched[id];
                if (any || !add_old) {
                    float* dst = dwte + (size_t)v * C;
                    #pragma unroll
                    for (int i = 0; i < WTE_MAXP; i++) {
                        const int p = pbase + lane + 32 * i;
                        if (p < npack) {
                            f32x4 o = acc[i];
                            if (add_old) {
                                const f32x4 old = ld128(dst + p * 4);
                                #pragma unroll
                                for (int e = 0; e < 4; e++) o[e] += old[e];
                            }
                            st128(dst + p * 4, o);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) touched[id] = 1;
        }
        __syncthreads();
        if (threadIdx.x == 0) list_len = 0;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// LayerNorm

// One warp per row.  With inp2 the row is inp1 + inp2 and is stored to `residual` first (the fused residual form).
__global__ void __launch_bounds__(256)
ln_fwd_f32(float* __restrict__ out, float* __restrict__ mean_out, float* __restrict__ rstd_out, float* __restrict__ residual,
           const float* __restrict__ inp1, const float* __restrict__ inp2, const float* __restrict__ weight,
           const float* __restrict__ bias, int rows, int C) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int npack = C >> 2;
    const float* x1 = inp1 + row * C;
    const float* x = x1;
    if (inp2 != nullptr) {
        const float* x2 = inp2 + row * C;
        float* r = residual + row * C;
        for (int p = lane; p < npack; p += 32) {
            f32x4 a = ld128cs(x1 + p * 4);
            const f32x4 b = ld128cs(x2 + p * 4);
            #pragma unroll
            for (int e = 0; e < 4; e++) a[e] += b[e];
            st128(r + p * 4, a);
        }
        __syncwarp();
        x = r;                                   // re-read what this warp just wrote (same lanes, same addresses)
    }
    float s = 0.f;
    for (int p = lane; p < npack; p += 32) {
        const f32x4 a = ld128(x + p * 4);
        s += (a[0] + a[1]) + (a[2] + a[3]);
    }
    const float mean = warp_sum(s) / C;
    float v = 0.f;
    for (int p = lane; p < npack; p += 32) {
        const f32x4 a = ld128(x + p * 4);
        #pragma unroll
        for (int e = 0; e < 4; e++) { const float d = a[e] - mean; v += d * d; }
    }
    const float rstd = rsqrtf(warp_sum(v) / C + 1e-5f);
    float* o = out + row * C;
    for (int p = lane; p < npack; p += 32) {
        const f32x4 a = ld128(x + p * 4), w = ld128(weight + p * 4), b = ld128(bias + p * 4);
        f32x4 y;
        #pragma unroll
        for (int e = 0; e < 4; e++) y[e] = (a[e] - mean) * rstd * w[e] + b[e];
        st128cs(o + p * 4, y);
    }
    if (lane == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
    }
}

constexpr int LNB_MAXP = 8;          // float4 packs per lane and pass: 1024 channels per pass
constexpr int LNB_WARPS = 8;

// Backward: dinp (+)= ..., and per-warp partial sums of dweight, dbias and (optionally) of the columns of the final dinp,
// written to `partials` as [3][total warps][C]; ln_bwd_fold_f32 adds them in warp order.  A warp walks rows
// warp_id, warp_id + total_warps, ...; channels beyond 1024 are handled in further passes over the same rows.
__global__ void __launch_bounds__(LNB_WARPS * 32)
ln_bwd_f32(float* __restrict__ dinp, float* __restrict__ partials, const float* __restrict__ dout, const float* __restrict__ inp,
           const float* __restrict__ weight, const float* __restrict__ mean, const float* __restrict__ rstd,
           int rows, int C, int accumulate_dinp, int want_colsum) {
    const int lane = threadIdx.x & 31;
    const int wid = blockIdx.x * LNB_WARPS + (threadIdx.x >> 5), nw = gridDim.x * LNB_WARPS;
    const int npack = C >> 2;
    for (int pbase = 0; pbase < npack; pbase += 32 * LNB_MAXP) {
        f32x4 dw[LNB_MAXP], db[LNB_MAXP], dc[LNB_MAXP];
        #pragma unroll
        for (int i = 0; i < LNB_MAXP; i++) { dw[i] = f32x4::zeros(); db[i] = f32x4::zeros(); dc[i] = f32x4::zeros(); }
        for (long long row = wid; row < rows; row += nw) {
            const float* dy = dout + row * C;
            const float* x = inp + row * C;
            const float m = mean[row], rs = rstd[row];
            // the two row means over ALL channels
            float s1 = 0.f, s2 = 0.f;
            for (int p = lane; p < npack; p += 32) {
                const f32x4 g = ld128(dy + p * 4), a = ld128(x + p * 4), w = ld128(weight + p * 4);
                #pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float dn = g[e] * w[e];
                    s1 += dn;
                    s2 += dn * (a[e] - m) * rs;
                }
            }
            s1 = warp_sum(s1) / C;
            s2 = warp_sum(s2) / C;
            float* dx = dinp + row * C;
            #pragma unroll
            for (int i = 0; i < LNB_MAXP; i++) {
                const int p = pbase + lane + 32 * i;
                if (p < npack) {
                    const f32x4 g = ld128(dy + p * 4), a = ld128(x + p * 4), w = ld128(weight + p * 4);
                    f32x4 o;
                    if (accumulate_dinp) o = ld128(dx + p * 4); else o = f32x4::zeros();
                    #pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float n = (a[e] - m) * rs;
                        const float dn = g[e] * w[e];
                        dw[i][e] += g[e] * n;
                        db[i][e] += g[e];
                        o[e] += (dn - s1 - n * s2) * rs;
                        dc[i][e] += o[e];
                    }
                    st128(dx + p * 4, o);
                }
            }
        }
        #pragma unroll
        for (int i = 0; i < LNB_MAXP; i++) {
            const int p = pbase + lane + 32 * i;
            if (p < npack) {
                st128(partials + ((size_t)0 * nw + wid) * C + p * 4, dw[i]);
                st128(partials + ((size_t)1 * nw + wid) * C + p * 4, db[i]);
                if (want_colsum) st128(partials + ((size_t)2 * nw + wid) * C + p * 4, dc[i]);
            }
        }
    }
}

// dst[c] (+)= sum over w (ascending) of partials[which][w][c] for the three destinations (null: skipped)
__global__ void ln_bwd_fold_f32(float* __restrict__ dweight, float* __restrict__ dbias, float* __restrict__ dcolsum,
                                const float* __restrict__ partials, int nw, int C, int acc_dwdb, int acc_dcol) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float* dst[3] = {dweight, dbias, dcolsum};
    const int acc[3] = {acc_dwdb, acc_dwdb, acc_dcol};
    #pragma unroll
    for (int k = 0; k < 3; k++) {
        if (dst[k] == nullptr) continue;
        float s = 0.f;
        for (int w = 0; w < nw; w++) s += partials[((size_t)k * nw + w) * C + c];
        if (acc[k]) s += dst[k][c];
        dst[k][c] = s;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// bias gradient: column sums of dout[rows, OC]; strips of rows -> partials[strip][OC] -> fold in strip order

__global__ void __launch_bounds__(256)
bias_grad_f32(float* __restrict__ partials, const float* __restrict__ dout, int rows, int OC, int rows_per_strip) {
    __shared__ float sh[8][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 128 + lane * 4;
    const int r0 = blockIdx.y * rows_per_strip, r1 = min(rows, r0 + rows_per_strip);
    f32x4 acc = f32x4::zeros();
    if (col < OC) {
        for (int r = r0 + warp; r < r1; r += 8) {
            const f32x4 d = ld128cs(dout + (size_t)r * OC + col);
            #pragma unroll
            for (int e = 0; e < 4; e++) acc[e] += d[e];
        }
    }
    #pragma unroll
    for (int e = 0; e < 4; e++) sh[warp][lane * 4 + e] = acc[e];
    __syncthreads();
    const int c = threadIdx.x;
    if (c < 128 && blockIdx.x * 128 + c < OC) {
        float s = 0.f;
        #pragma unroll
        for (int w = 0; w < 8; w++) s += sh[w][c];
        partials[(size_t)blockIdx.y * OC + blockIdx.x * 128 + c] = s;
    }
}

__global__ void bias_grad_fold_f32(float* __restrict__ dbias, const float* __restrict__ partials, int strips, int OC, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= OC) return;
    float s = 0.f;
    for (int i = 0; i < strips; i++) s += partials[(size_t)i * OC + c];
    if (accumulate) s += dbias[c];
    dbias[c] = s;
}

// ---------------------------------------------------------------------------------------------------------------------
// classifier: softmax + cross-entropy over logits[rows, Vp] (first V columns are real); the logits are replaced by their gradient

__global__ void __launch_bounds__(256)
classifier_f32(float* __restrict__ logits, float* __restrict__ losses, const int* __restrict__ targets, float dloss,
               int V, int Vp, int write_dlogits, int accumulate_loss) {
    __shared__ float red[32];
    float* x = logits + (size_t)blockIdx.x * Vp;
    if (threadIdx.x == 0) (void)LLMC_DBG_CHECK(targets[blockIdx.x] >= 0 && targets[blockIdx.x] < V, 0xC01);
    const int target = min(max(targets[blockIdx.x], 0), V - 1);
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, red);
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(x[i] - mx);
    s = block_sum(s, red);
    const float xt = x[target];
    __syncthreads();                                        // every thread has read x[target] before anyone overwrites it
    if (threadIdx.x == 0) {
        const float loss = logf(s) + mx - xt;
        losses[blockIdx.x] = accumulate_loss ? losses[blockIdx.x] + loss : loss;
    }
    if (write_dlogits) {
        const float inv = 1.0f / s;
        for (int i = threadIdx.x; i < Vp; i += blockDim.x) {
            float g = 0.f;
            if (i < V) g = (expf(x[i] - mx) * inv - (i == target ? 1.0f : 0.0f)) * dloss;
            x[i] = g;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// attention pieces

// qkv[B, T, 3, NH, HS]  <->  sep[3, B * NH, T, HS]   (to_sep = 1: split and permute; 0: the inverse, for the gradients)
__global__ void permute_qkv_f32(float* __restrict__ sep, float* __restrict__ qkv, int B, int T, int NH, int HS, int to_sep) {
    const int hp = HS >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)B * T * 3 * NH * hp;
    if (idx >= total) return;
    long long r = idx;
    const int p = (int)(r % hp); r /= hp;
    const int h = (int)(r % NH); r /= NH;
    const int w = (int)(r % 3); r /= 3;
    const int t = (int)(r % T);
    const int b = (int)(r / T);
    float* a = qkv + idx * 4;
    float* s = sep + ((((size_t)w * B + b) * NH + h) * T + t) * HS + p * 4;
    if (to_sep) st128(s, ld128cs(a)); else st128(a, ld128cs(s));
}

// y[B, NH, T, HS]  <->  out[B, T, NH, HS]   (to_out = 1: y -> out; 0: out -> y)
__global__ void permute_heads_f32(float* __restrict__ y, float* __restrict__ out, int B, int T, int NH, int HS, int to_out) {
    const int hp = HS >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)B * T * NH * hp;
    if (idx >= total) return;
    long long r = idx;
    const int p = (int)(r % hp); r /= hp;
    const int h = (int)(r % NH); r /= NH;
    const int t = (int)(r % T);
    const int b = (int)(r / T);
    float* o = out + idx * 4;
    float* s = y + ((((size_t)b * NH + h) * T + t)) * HS + p * 4;
    if (to_out) st128(o, ld128cs(s)); else st128(s, ld128cs(o));
}

// att[bh, t, :] (scores q.k, unscaled) -> causal softmax of scale * scores, in place; lse[bh, t] = log of the row's sum of
// exponentials (of the scaled scores).  With lse_in the row is normalised by that stored value instead (backward pass).
// One warp per row.
__global__ void __launch_bounds__(256)
softmax_causal_f32(float* __restrict__ att, float* __restrict__ lse_out, const float* __restrict__ lse_in, float scale, long long rows, int T) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int t = (int)(row % T);
    float* x = att + row * T;
    float l;
    if (lse_in != nullptr) {
        l = lse_in[row];
    } else {
        float mx = -INFINITY;
        for (int j = lane; j <= t; j += 32) mx = fmaxf(mx, x[j] * scale);
        mx = warp_max(mx);
        float s = 0.f;
        for (int j = lane; j <= t; j += 32) s += expf(x[j] * scale - mx);
        s = warp_sum(s);
        l = logf(s) + mx;
        if (lane == 0) lse_out[row] = l;
    }
    for (int j = lane; j < T; j += 32) x[j] = (j <= t) ? expf(x[j] * scale - l) : 0.f;
}

// datt[bh, t, j] = scale * p[t, j] * (datt[t, j] - sum_k p[t, k] datt[t, k]) for j <= t, 0 beyond; in place.  One warp per row.
__global__ void __launch_bounds__(256)
softmax_causal_bwd_f32(float* __restrict__ datt, const float* __restrict__ att, float scale, long long rows, int T) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int t = (int)(row % T);
    float* d = datt + row * T;
    const float* p = att + row * T;
    float s = 0.f;
    for (int j = lane; j <= t; j += 32) s += p[j] * d[j];
    s = warp_sum(s);
    for (int j = lane; j < T; j += 32) d[j] = (j <= t) ? scale * p[j] * (d[j] - s) : 0.f;
}

// ---------------------------------------------------------------------------------------------------------------------
// optimizer

// One tensor of L slices: parameters at params[p_base + l * p_stride + i], optimizer state at [o_base + l * o_stride + i].
// The clip coefficient comes from the squared norm on the device; a non-finite norm leaves everything untouched.
__global__ void adamw_f32(float* __restrict__ params, float* __restrict__ master, const float* __restrict__ grads,
                          float* __restrict__ m, float* __restrict__ v, long long p_base, long long p_stride, long long o_base,
                          long long o_stride, long long n, float lr, float beta1, float beta2, float bc1, float bc2, float eps,
                          float wd, float grad_scale, const float* __restrict__ norm_sq, float grad_clip) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float scale = grad_scale;
    if (norm_sq != nullptr) {
        const float nsq = norm_sq[0];
        if (!isfinite(nsq)) return;
        const float nrm = sqrtf(nsq);
        if (nrm > grad_clip) scale = grad_scale * grad_clip / nrm;
    }
    const long long pi = p_base + (long long)blockIdx.y * p_stride + i, oi = o_base + (long long)blockIdx.y * o_stride + i;
    const float g = grads[pi] * scale;
    const float mm = beta1 * m[oi] + (1.0f - beta1) * g;
    const float vv = beta2 * v[oi] + (1.0f - beta2) * g * g;
    m[oi] = mm;
    v[oi] = vv;
    const float old = master != nullptr ? master[oi] : params[pi];
    const float nw = old - lr * ((mm / bc1) / (sqrtf(vv / bc2) + eps) + wd * old);
    params[pi] = nw;
    if (master != nullptr) master[oi] = nw;
}

constexpr int SUMSQ_CTAS = 64;
// partials[blockIdx.y * SUMSQ_CTAS + blockIdx.x] = sum of squares of this CTA's share of slice blockIdx.y (fixed order)
__global__ void __launch_bounds__(256)
sumsq_f32(float* __restrict__ partials, const float* __restrict__ x, long long base, long long stride, long long n) {
    __shared__ float red[32];
    const float* p = x + base + (long long)blockIdx.y * stride;
    float s = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) s += p[i] * p[i];
    s = block_sum(s, red);
    if (threadIdx.x == 0) partials[(size_t)blockIdx.y * SUMSQ_CTAS + blockIdx.x] = s;
}

__global__ void copy_f32(float* __restrict__ dst, const float* __restrict__ src, long long d_base, long long d_stride, long long s_base,
                         long long s_stride, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    dst[d_base + (long long)blockIdx.y * d_stride + i] = src[s_base + (long long)blockIdx.y * s_stride + i];
}

}  // namespace

#define GRID1(total, threads) (unsigned)CEIL_DIV((long long)(total), (long long)(threads))

static int aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int llmc_f32_gelu_fwd(float* out, const float* inp, long long n, cudaStream_t stream) {
    if (n % 4 || !aligned16(out) || !aligned16(inp)) return -1;
    gelu_fwd_f32<<<GRID1(n / 4, 256), 256, 0, stream>>>(out, inp, n / 4);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_gelu_bwd(float* d_inout, const float* inp, long long n, cudaStream_t stream) {
    if (n % 4 || !aligned16(d_inout) || !aligned16(inp)) return -1;
    gelu_bwd_f32<<<GRID1(n / 4, 256), 256, 0, stream>>>(d_inout, inp, n / 4);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_residual_add(float* out, const float* a, const float* b, long long n, cudaStream_t stream) {
    if (n % 4 || !aligned16(out) || !aligned16(a) || !aligned16(b)) return -1;
    residual_add_f32<<<GRID1(n / 4, 256), 256, 0, stream>>>(out, a, b, n / 4);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_encoder_fwd(float* out, const int* tokens, const float* wte, const float* wpe, int B, int T, int C, int V,
                                    cudaStream_t stream) {
    if (C % 4 || !aligned16(out) || !aligned16(wte) || !aligned16(wpe)) return -1;
    encoder_fwd_f32<<<GRID1((long long)B * T * (C / 4), 256), 256, 0, stream>>>(out, tokens, wte, wpe, B, T, C, V);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// accumulate_* = 0: the table is overwritten (rows of dwte without any hit become zero); 1: added to.
extern "C" int llmc_f32_encoder_bwd(float* dwte, float* dwpe, const float* dout, const int* tokens, int B, int T, int C, int V,
                                    int accumulate_wte, int accumulate_wpe, cudaStream_t stream) {
    if (C % 4 || !aligned16(dwte) || !aligned16(dwpe) || !aligned16(dout)) return -1;
    if (dwpe != nullptr) {
        wpe_bwd_f32<<<GRID1(T * (C / 4), 256), 256, 0, stream>>>(dwpe, dout, B, T, C, accumulate_wpe);
        CUDA_CHECK(cudaGetLastError());
    }
    wte_bwd_f32<<<CEIL_DIV(V, IDS_PER_CTA), WTE_THREADS, 0, stream>>>(dwte, dout, tokens, B * T, C, V, accumulate_wte);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// out = LayerNorm(inp1 [+ inp2]); with inp2 the sum is stored to `residual`.  mean / rstd may be null.
extern "C" int llmc_f32_layernorm_fwd(float* out, float* mean, float* rstd, float* residual, const float* inp1, const float* inp2,
                                      const float* weight, const float* bias, int rows, int C, cudaStream_t stream) {
    if (C % 4 || !aligned16(out) || !aligned16(inp1) || !aligned16(inp2) || !aligned16(residual) || !aligned16(weight) || !aligned16(bias)) return -1;
    if (inp2 != nullptr && residual == nullptr) return -1;
    ln_fwd_f32<<<GRID1(rows, 8), 256, 0, stream>>>(out, mean, rstd, residual, inp1, inp2, weight, bias, rows, C);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

static int lnb_ctas(int rows) {
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int ctas = 2 * sms;
    const int need = CEIL_DIV(rows, LNB_WARPS);
    return need < ctas ? (need > 0 ? need : 1) : ctas;
}

// floats of scratch the backward needs: three partial tables of [warps][C]
extern "C" long long llmc_f32_layernorm_bwd_scratch(int rows, int C) { return 3ll * lnb_ctas(rows) * LNB_WARPS * C; }

extern "C" int llmc_f32_layernorm_bwd(float* dinp, float* dweight, float* dbias, float* dcolsum, float* scratch, const float* dout,
                                      const float* inp, const float* weight, const float* mean, const float* rstd, int rows, int C,
                                      int accumulate_dinp, int accumulate_dwdb, int accumulate_dcol, cudaStream_t stream) {
    if (C % 4 || !aligned16(dinp) || !aligned16(dout) || !aligned16(inp) || !aligned16(weight) || !aligned16(scratch)) return -1;
    const int ctas = lnb_ctas(rows);
    ln_bwd_f32<<<ctas, LNB_WARPS * 32, 0, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, rows, C, accumulate_dinp, dcolsum != nullptr);
    CUDA_CHECK(cudaGetLastError());
    ln_bwd_fold_f32<<<CEIL_DIV(C, 128), 128, 0, stream>>>(dweight, dbias, dcolsum, scratch, ctas * LNB_WARPS, C, accumulate_dwdb, accumulate_dcol);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

static int bgf_strips(int rows) {
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int strips = CEIL_DIV(rows, 64);
    return strips < 2 * sms ? (strips > 0 ? strips : 1) : 2 * sms;
}

extern "C" long long llmc_f32_bias_grad_scratch(int rows, int OC) { return (long long)bgf_strips(rows) * OC; }

extern "C" int llmc_f32_bias_grad(float* dbias, float* scratch, const float* dout, int rows, int OC, int accumulate, cudaStream_t stream) {
    if (OC % 4 || !aligned16(dout)) return -1;
    const int strips = bgf_strips(rows);
    const int rps = CEIL_DIV(rows, strips);
    bias_grad_f32<<<dim3(CEIL_DIV(OC, 128), strips), 256, 0, stream>>>(scratch, dout, rows, OC, rps);
    CUDA_CHECK(cudaGetLastError());
    bias_grad_fold_f32<<<CEIL_DIV(OC, 256), 256, 0, stream>>>(dbias, scratch, strips, OC, accumulate);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_classifier(float* logits, float* losses, const int* targets, float dloss, int rows, int V, int Vp,
                                   int write_dlogits, int accumulate_loss, cudaStream_t stream) {
    if (rows <= 0) return 0;
    classifier_f32<<<rows, 256, 0, stream>>>(logits, losses, targets, dloss, V, Vp, write_dlogits, accumulate_loss);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_permute_qkv(float* sep, float* qkv, int B, int T, int NH, int HS, int to_sep, cudaStream_t stream) {
    if (HS % 4 || !aligned16(sep) || !aligned16(qkv)) return -1;
    permute_qkv_f32<<<GRID1((long long)B * T * 3 * NH * (HS / 4), 256), 256, 0, stream>>>(sep, qkv, B, T, NH, HS, to_sep);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_permute_heads(float* y, float* out, int B, int T, int NH, int HS, int to_out, cudaStream_t stream) {
    if (HS % 4 || !aligned16(y) || !aligned16(out)) return -1;
    permute_heads_f32<<<GRID1((long long)B * T * NH * (HS / 4), 256), 256, 0, stream>>>(y, out, B, T, NH, HS, to_out);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// lse_in null: forward (writes lse_out); else the rows are normalised with the stored values (backward recomputation)
extern "C" int llmc_f32_softmax_causal(float* att, float* lse_out, const float* lse_in, float scale, long long rows, int T, cudaStream_t stream) {
    softmax_causal_f32<<<GRID1(rows, 8), 256, 0, stream>>>(att, lse_out, lse_in, scale, rows, T);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_softmax_causal_bwd(float* datt, const float* att, float scale, long long rows, int T, cudaStream_t stream) {
    softmax_causal_bwd_f32<<<GRID1(rows, 8), 256, 0, stream>>>(datt, att, scale, rows, T);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_adamw(float* params, float* master, const float* grads, float* m, float* v, long long p_base, long long p_stride,
                              long long o_base, long long o_stride, long long n, int L, float lr, float beta1, float beta2, int t, float eps,
                              float wd, float grad_scale, const float* norm_sq, float grad_clip, cudaStream_t stream) {
    if (n <= 0 || L <= 0) return 0;
    const float bc1 = 1.0f - powf(beta1, (float)t), bc2 = 1.0f - powf(beta2, (float)t);
    adamw_f32<<<dim3(GRID1(n, 256), L), 256, 0, stream>>>(params, master, grads, m, v, p_base, p_stride, o_base, o_stride, n, lr, beta1, beta2,
                                                           bc1, bc2, eps, wd, grad_scale, norm_sq, grad_clip);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_sumsq_partials_per_slice() { return SUMSQ_CTAS; }

// partials: L * llmc_f32_sumsq_partials_per_slice() floats
extern "C" int llmc_f32_sumsq(float* partials, const float* x, long long base, long long stride, long long n, int L, cudaStream_t stream) {
    if (L <= 0) return 0;
    sumsq_f32<<<dim3(SUMSQ_CTAS, L), 256, 0, stream>>>(partials, x, base, stride, n);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_f32_copy_slices(float* dst, const float* src, long long d_base, long long d_stride, long long s_base, long long s_stride,
                                    long long n, int L, cudaStream_t stream) {
    if (n <= 0 || L <= 0) return 0;
    copy_f32<<<dim3(GRID1(n, 256), L), 256, 0, stream>>>(dst, src, d_base, d_stride, s_base, s_stride, n);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
