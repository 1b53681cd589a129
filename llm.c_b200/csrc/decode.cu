// Incremental decoding with a key / value cache (the inference path of the reference's LLaMA script,
// train_llama3.py:167-190 and :476-556: keys and values of earlier positions are kept, only the new tokens run through
// the network).  Two kernels; both are memory-bound and small, so they use plain loads, no tensor cores:
//
//   rope_cache      raw (N, (NH + 2 NKV) * HS), N = B * Tq new tokens at positions start_pos .. start_pos + Tq - 1
//                     -> q (N, NH, HS) rotated queries
//                     -> kcache / vcache (B, Tmax, NKV, HS): rotated keys and the values written at their positions
//   cached_attention  out (N, NH, HS) = softmax(q . K[0 .. pos] / sqrt(HS)) V[0 .. pos] per (batch row, new token, head);
//                     grouped queries read the cache head h / (NH / NKV) directly, nothing is expanded.
//
// start_pos comes from the host or, when `pos_ptr` is given, from device memory: a decoding step captured in a CUDA graph is
// replayed with the position advanced on the device.  A device position that would leave the cache or the rotary table makes
// the kernel record ST_BAD_ARG in the status word and return without touching memory.
#include "common.cuh"

namespace {

DEVINL bf16x8 rotate8(const bf16x8& a, const float4& cs0, const float4& cs1) {
    bf16x8 r;
    const float c[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
    const float s[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
    #pragma unroll
    for (int j = 0; j < 4; j++) {
        const float re = __bfloat162float(a[2 * j]), im = __bfloat162float(a[2 * j + 1]);
        r[2 * j] = __float2bfloat16_rn(re * c[j] - im * s[j]);
        r[2 * j + 1] = __float2bfloat16_rn(re * s[j] + im * c[j]);
    }
    return r;
}

__global__ void __launch_bounds__(256)
rope_cache_kernel(bf16* __restrict__ q, bf16* __restrict__ kcache, bf16* __restrict__ vcache, const bf16* __restrict__ raw,
                  const float2* __restrict__ freqs, long long N, int Tq, int Tmax, int start_pos, int NH, int NKV, int HS,
                  const int* __restrict__ pos_ptr, int freqs_len, unsigned int* status) {
    if (pos_ptr) {
        start_pos = *pos_ptr;
        if (start_pos < 0 || start_pos + Tq > Tmax || start_pos + Tq > freqs_len) {
            if (threadIdx.x == 0 && blockIdx.x == 0) record_error(status, ST_BAD_ARG, 0x30);
            return;
        }
    }
    const int hp = HS >> 3;
    const int heads = NH + 2 * NKV;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * heads * hp) return;
    const int p = (int)(idx % hp);
    const int h = (int)((idx / hp) % heads);
    const long long n = idx / ((long long)hp * heads);
    const int pos = start_pos + (int)(n % Tq);
    const long long b = n / Tq;
    bf16x8 a = ld128cs(raw + (n * heads + h) * HS + p * 8);
    if (h < NH + NKV) {
        const float4* f = reinterpret_cast<const float4*>(freqs + (size_t)pos * (HS >> 1) + p * 4);
        a = rotate8(a, f[0], f[1]);
    }
    if (h < NH) {
        st128(q + (n * NH + h) * HS + p * 8, a);
    } else if (h < NH + NKV) {
        st128(kcache + ((b * Tmax + pos) * NKV + (h - NH)) * HS + p * 8, a);
    } else {
        st128(vcache + ((b * Tmax + pos) * NKV + (h - NH - NKV)) * HS + p * 8, a);
    }
}

constexpr int DEC_THREADS = 128;
constexpr int DEC_CHUNK = 512;      // keys whose scores sit in shared memory at a time (running maximum across chunks)
constexpr int DEC_MAX_HS = 128;

// One CTA per (head, new token, batch row).  Scores: a thread per key, the query in shared memory as fp32 (already scaled).
// Weighted sum of the values: a thread per pair of channels, DEC_THREADS / (HS / 2) key groups side by side, folded at the end.
__global__ void __launch_bounds__(DEC_THREADS)
cached_attention_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ kcache,
                        const bf16* __restrict__ vcache, int Tq, int Tmax, int start_pos, int NH, int NKV, int HS, float scale,
                        const int* __restrict__ pos_ptr, unsigned int* status) {
    if (pos_ptr) {
        start_pos = *pos_ptr;
        if (start_pos < 0 || start_pos + Tq > Tmax) {
            if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) record_error(status, ST_BAD_ARG, 0x31);
            return;
        }
    }
    __shared__ float qs[DEC_MAX_HS];
    __shared__ float sc[DEC_CHUNK];
    __shared__ float red[32];
    __shared__ float part[DEC_THREADS * 2];
    const int tid = threadIdx.x;
    const int h = blockIdx.x, t = blockIdx.y;
    const long long b = blockIdx.z;
    const long long n = b * Tq + t;
    const int g = h / (NH / NKV);
    const int nkeys = start_pos + t + 1;
    if (tid < HS) qs[tid] = __bfloat162float(q[(n * NH + h) * HS + tid]) * scale;
    __syncthreads();
    const int pairs = HS >> 1;
    const int groups = DEC_THREADS / pairs;
    const int my_pair = tid % pairs, my_group = tid / pairs;
    const int hp = HS >> 3;
    float m = -INFINITY, l = 0.f, acc0 = 0.f, acc1 = 0.f;
    for (int base = 0; base < nkeys; base += DEC_CHUNK) {
        const int cnt = min(DEC_CHUNK, nkeys - base);
        float lmax = -INFINITY;
        for (int j = tid; j < cnt; j += DEC_THREADS) {
            const bf16* krow = kcache + ((b * Tmax + base + j) * NKV + g) * HS;
            float s = 0.f;
            #pragma unroll 4
            for (int p = 0; p < hp; p++) {                    // four independent 128-bit loads in flight per thread
                const bf16x8 kk = ld128(krow + p * 8);
                #pragma unroll
                for (int e = 0; e < 8; e++) s += qs[p * 8 + e] * __bfloat162float(kk[e]);
            }
            sc[j] = s;
            lmax = fmaxf(lmax, s);
        }
        const float m_new = fmaxf(m, block_max(lmax, red));
        float lsum = 0.f;
        for (int j = tid; j < cnt; j += DEC_THREADS) {
            const float pj = __expf(sc[j] - m_new);
            sc[j] = pj;
            lsum += pj;
        }
        const float csum = block_sum(lsum, red);
        const float corr = __expf(m - m_new);
        l = l * corr + csum;
        acc0 *= corr;
        acc1 *= corr;
        m = m_new;
        if (my_group < groups) {
            #pragma unroll 8
            for (int j = my_group; j < cnt; j += groups) {
                const bf16* vrow = vcache + ((b * Tmax + base + j) * NKV + g) * HS;
                const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vrow + 2 * my_pair));
                acc0 += sc[j] * vv.x;
                acc1 += sc[j] * vv.y;
            }
        }
        __syncthreads();
    }
    part[tid * 2] = (my_group < groups) ? acc0 : 0.f;
    part[tid * 2 + 1] = (my_group < groups) ? acc1 : 0.f;
    __syncthreads();
    if (tid < pairs) {
        float o0 = 0.f, o1 = 0.f;
        for (int gi = 0; gi < groups; gi++) {
            o0 += part[(gi * pairs + tid) * 2];
            o1 += part[(gi * pairs + tid) * 2 + 1];
        }
        const float inv = 1.0f / l;
        *reinterpret_cast<__nv_bfloat162*>(out + (n * NH + h) * HS + 2 * tid) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Decoding attention, fast path (head width 64 or 128, at most 8 query rows per cached head: the decoding step itself).
// The general kernel above gives a thread a whole key row straight from global memory (32 rows per load instruction, one
// cache line each) and runs once per QUERY head, so grouped queries re-read their keys; it is bound by instruction issue at
// a fifth of the memory rate.  Here
//   * a CTA serves ONE cached head of one batch row for ALL its R = (NH / NKV) * Tq query rows and a slice of the keys
//     (grid: key slices x cached heads x batch rows, sized to fill the GPU at any batch size);
//   * each of its 4 warps walks tiles of 32 keys.  The K tile comes in with cp.async (16 lanes read one 256-byte row:
//     coalesced), double buffered, into shared memory with the 16-byte chunks of row j XOR-swizzled by j & 7; then lane j
//     owns key j and reads its row without bank conflicts: whole dot products per lane, no butterflies, one exponential
//     per key and query row;
//   * the probabilities go through a small shared tile; for the weighted sum of V every lane owns HS / 32 channels and the
//     V rows are read from global memory as the 32 lanes' contiguous 8- or 4-byte pieces, eight rows in flight;
//   * running (max, sum, accumulator) per warp, merged over the warps, then over the key slices in a small fp32 workspace
//     that a second kernel folds in slice order (deterministic).
constexpr int CA_WARPS = 4;
constexpr int CA_THREADS = CA_WARPS * 32;
constexpr int CA_MAX_R = 8;
constexpr int CA_MIN_KEYS = 256;      // a slice is at least this long (unless the cache is shorter)
constexpr float CA_LOG2E = 1.4426950408889634f;

DEVINL void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
DEVINL void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> DEVINL void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int HS_, int R> constexpr int ca_smem_bytes() {
    return R * HS_ * 4 + CA_WARPS * (2 * 32 * HS_ * 2 + 32 * R * 4);
}

template <int HS_, int R>
__global__ void __launch_bounds__(CA_THREADS)
cached_attention_split_kernel(float* __restrict__ ws, const bf16* __restrict__ q, const bf16* __restrict__ kcache,
                              const bf16* __restrict__ vcache, int Tq, int Tmax, int start_pos, int NH, int NKV, float scale,
                              const int* __restrict__ pos_ptr, unsigned int* status, int keys_per_slice, int rows) {
    if (pos_ptr) {
        start_pos = *pos_ptr;
        if (start_pos < 0 || start_pos + Tq > Tmax) {
            if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) record_error(status, ST_BAD_ARG, 0x32);
            return;
        }
    }
    constexpr int ROWB = HS_ * 2;              // bytes of a key row
    constexpr int CHUNKS = HS_ / 8;            // 16-byte chunks of a row
    constexpr int CPL = HS_ / 32;              // channels of V and of the output per lane
    extern __shared__ __align__(16) uint8_t ca_smem[];
    float* qs = reinterpret_cast<float*>(ca_smem);                                   // [R][HS_], scaled by scale * log2(e)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* kbuf = ca_smem + R * HS_ * 4 + warp * (2 * 32 * ROWB + 32 * R * 4);      // [2][32 rows][ROWB], swizzled
    float* ptile = reinterpret_cast<float*>(kbuf + 2 * 32 * ROWB);                   // [32 keys][R]
    const int slice = blockIdx.x, g = blockIdx.y, nslices = gridDim.x;
    const long long b = blockIdx.z;
    const int G = NH / NKV;
    const int nkeys = start_pos + Tq;                          // keys visible to the last new token
    const int k0 = slice * keys_per_slice, k1 = min(nkeys, k0 + keys_per_slice);

    // query rows: r -> token r / G, head g * G + r % G; rows past `rows` repeat row 0 and are dropped at the end
    for (int i = threadIdx.x; i < R * HS_; i += CA_THREADS) {
        const int r = i / HS_, c = i - r * HS_;
        const int rr = r < rows ? r : 0;
        const int t = rr / G, hq = g * G + rr % G;
        qs[i] = __bfloat162float(q[((b * Tq + t) * NH + hq) * HS_ + c]) * (scale * CA_LOG2E);
    }
    int limit[R];                                              // keys [0, limit) are visible to row r
    #pragma unroll
    for (int r = 0; r < R; r++) limit[r] = min(k1, start_pos + (r < rows ? r : 0) / G + 1);
    __syncthreads();

    float m[R], l[R], acc[R][CPL];
    #pragma unroll
    for (int r = 0; r < R; r++) {
        m[r] = -INFINITY; l[r] = 0.f;
        #pragma unroll
        for (int c = 0; c < CPL; c++) acc[r][c] = 0.f;
    }
    const long long row_stride = (long long)NKV * HS_;
    const bf16* kbase = kcache + ((b * Tmax) * NKV + g) * HS_;
    const bf16* vbase = vcache + ((b * Tmax) * NKV + g) * HS_ + lane * CPL;
    // copy of the K tile that starts at key kt into buffer `which` (rows past k1 are not copied and never used)
    auto fetch = [&](int kt, int which) {
        uint8_t* dst = kbuf + which * 32 * ROWB;
        #pragma unroll
        for (int i = 0; i < CHUNKS; i++) {
            const int qid = i * 32 + lane, row = qid / CHUNKS, c = qid % CHUNKS;
            if (kt + row < k1) cp_async16(dst + row * ROWB + ((c ^ (row & 7)) * 16), kbase + (kt + row) * row_stride + c * 8);
        }
        cp_async_commit();
    };
    constexpr int TSTEP = CA_WARPS * 32;
    const int kt0 = k0 + warp * 32;
    if (kt0 < k1) fetch(kt0, 0);
    int buf = 0;
    for (int kt = kt0; kt < k1; kt += TSTEP, buf ^= 1) {
        if (kt + TSTEP < k1) { fetch(kt + TSTEP, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncwarp();
        // ---- scores: lane j owns key kt + j
        const uint8_t* krow = kbuf + buf * 32 * ROWB + lane * ROWB;
        float s[R];
        #pragma unroll
        for (int r = 0; r < R; r++) s[r] = 0.f;
        #pragma unroll 4
        for (int c = 0; c < CHUNKS; c++) {
            const uint4 kq = *reinterpret_cast<const uint4*>(krow + ((c ^ (lane & 7)) * 16));
            const uint32_t ku[4] = {kq.x, kq.y, kq.z, kq.w};
            float kf[8];
            #pragma unroll
            for (int e = 0; e < 4; e++) { kf[2 * e] = __uint_as_float(ku[e] << 16); kf[2 * e + 1] = __uint_as_float(ku[e] & 0xffff0000u); }
            #pragma unroll
            for (int r = 0; r < R; r++) {
                const float4 qa = *reinterpret_cast<const float4*>(qs + r * HS_ + c * 8), qb = *reinterpret_cast<const float4*>(qs + r * HS_ + c * 8 + 4);
                s[r] = fmaf(qa.x, kf[0], s[r]); s[r] = fmaf(qa.y, kf[1], s[r]); s[r] = fmaf(qa.z, kf[2], s[r]); s[r] = fmaf(qa.w, kf[3], s[r]);
                s[r] = fmaf(qb.x, kf[4], s[r]); s[r] = fmaf(qb.y, kf[5], s[r]); s[r] = fmaf(qb.z, kf[6], s[r]); s[r] = fmaf(qb.w, kf[7], s[r]);
            }
        }
        // ---- running softmax of the tile (base 2: the queries carry log2(e))
        #pragma unroll
        for (int r = 0; r < R; r++) {
            const float sv = (kt + lane < limit[r]) ? s[r] : -INFINITY;
            const float mn = fmaxf(m[r], warp_max(sv));
            const float pj = (sv == -INFINITY) ? 0.f : ex2_fast(sv - mn);
            const float corr = (m[r] == -INFINITY) ? 0.f : ex2_fast(m[r] - mn);     // mn is finite whenever any key was visible
            if (mn != -INFINITY) {
                l[r] = l[r] * corr + warp_sum(pj);
                #pragma unroll
                for (int c = 0; c < CPL; c++) acc[r][c] *= corr;
                m[r] = mn;
            }
            ptile[lane * R + r] = pj;
        }
        __syncwarp();
        // ---- weighted sum of the V rows: lane owns channels lane * CPL .. + CPL - 1; eight rows in flight
        const int nv = min(32, k1 - kt);
        for (int i0 = 0; i0 < nv; i0 += 8) {
            uint32_t vr[8][CPL / 2];
            #pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u;
                #pragma unroll
                for (int w = 0; w < CPL / 2; w++) vr[u][w] = 0u;
                if (i < nv) {
                    const bf16* vp = vbase + (long long)(kt + i) * row_stride;
                    if (CPL == 4) { const uint2 t2 = __ldcs(reinterpret_cast<const uint2*>(vp)); vr[u][0] = t2.x; vr[u][CPL / 2 - 1] = t2.y; }
                    else vr[u][0] = __ldcs(reinterpret_cast<const unsigned int*>(vp));
                }
            }
            #pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u;
                if (i < nv) {                                   // uniform over the warp
                    float vf[CPL];
                    #pragma unroll
                    for (int w = 0; w < CPL / 2; w++) { vf[2 * w] = __uint_as_float(vr[u][w] << 16); vf[2 * w + 1] = __uint_as_float(vr[u][w] & 0xffff0000u); }
                    #pragma unroll
                    for (int r = 0; r < R; r++) {
                        const float pr = ptile[i * R + r];
                        #pragma unroll
                        for (int c = 0; c < CPL; c++) acc[r][c] = fmaf(pr, vf[c], acc[r][c]);
                    }
                }
            }
        }
        __syncwarp();                                           // the probability tile is rewritten by the next tile
    }
    // ---- merge the warps (the K buffers are free now): partial of this slice -> ws[((b, g), slice)][r][HS + 2]
    __syncthreads();
    float* sm_m = reinterpret_cast<float*>(ca_smem + R * HS_ * 4);                   // [CA_WARPS][R]
    float* sm_l = sm_m + CA_WARPS * R;
    float* sm_acc = sm_l + CA_WARPS * R;                                             // [CA_WARPS][R][HS_]
    #pragma unroll
    for (int r = 0; r < R; r++) {
        if (lane == 0) { sm_m[warp * R + r] = m[r]; sm_l[warp * R + r] = l[r]; }
        #pragma unroll
        for (int c = 0; c < CPL; c++) sm_acc[(warp * R + r) * HS_ + lane * CPL + c] = acc[r][c];
    }
    __syncthreads();
    float* dst = ws + (((size_t)(b * NKV + g) * nslices + slice) * R) * (HS_ + 2);
    for (int i = threadIdx.x; i < R * HS_; i += CA_THREADS) {
        const int r = i / HS_, c = i - r * HS_;
        float mn = -INFINITY;
        #pragma unroll
        for (int w = 0; w < CA_WARPS; w++) mn = fmaxf(mn, sm_m[w * R + r]);
        float a = 0.f, ls = 0.f;
        #pragma unroll
        for (int w = 0; w < CA_WARPS; w++) {
            const float mw = sm_m[w * R + r];
            const float cw = (mw == -INFINITY) ? 0.f : ex2_fast(mw - mn);
            a += sm_acc[(w * R + r) * HS_ + c] * cw;
            ls += sm_l[w * R + r] * cw;
        }
        dst[r * (HS_ + 2) + c] = a;
        if (c == 0) { dst[r * (HS_ + 2) + HS_] = mn; dst[r * (HS_ + 2) + HS_ + 1] = ls; }
    }
}

// out[row r of (b, g)] = sum over slices of acc_s * exp(m_s - M) / sum over slices of l_s * exp(m_s - M), slices in order
template <int HS_>
__global__ void cached_attention_combine_kernel(bf16* __restrict__ out, const float* __restrict__ ws, int Tq, int NH, int NKV,
                                                int nslices, int R, int rows) {
    const int r = blockIdx.x, g = blockIdx.y;
    const long long b = blockIdx.z;
    const int c = threadIdx.x;
    if (r >= rows || c >= HS_) return;
    const float* src = ws + ((size_t)(b * NKV + g) * nslices * R + r) * (HS_ + 2);
    const size_t sstride = (size_t)R * (HS_ + 2);
    float mn = -INFINITY;
    for (int s = 0; s < nslices; s++) mn = fmaxf(mn, src[s * sstride + HS_]);
    float a = 0.f, ls = 0.f;
    for (int s = 0; s < nslices; s++) {
        const float ms = src[s * sstride + HS_];
        const float cw = (ms == -INFINITY) ? 0.f : ex2_fast(ms - mn);        // the maxima are in base-2 units
        a += src[s * sstride + c] * cw;
        ls += src[s * sstride + HS_ + 1] * cw;
    }
    const int G = NH / NKV;
    const int t = r / G, hq = g * G + r % G;
    out[((b * Tq + t) * NH + hq) * HS_ + c] = __float2bfloat16_rn(a / ls);
}

// ---------------------------------------------------------------------------------------------------------------
// Skinny product for decoding steps: out (M, N) = x (M, K) . w (N, K)^T with M <= 8 rows.  A 128-row tcgen05 tile would
// spend its time on padding and, worse, leave most SMs without a tile (N / 128 tiles for 148 SMs), while the step is bound by
// streaming the weights once.  Here a CTA owns 16 output columns and its 8 warps split K; a warp feeds warp-level
// m16n8k16 MMAs with the weights as the 16-row operand and the (at most 8) activation rows as the 8-column operand, so that
// the arithmetic costs two instructions per KB of weights and the loop is nothing but 128-bit streaming loads.  A lane
// loads 8 consecutive K elements of weight rows g and g + 8 and of activation row g (g = lane / 4) and uses them as the
// K slots of two MMAs; the dot product does not care that this permutes K, as long as both operands agree.
constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_COLS = 16;
constexpr int SK_UNROLL = 4;
constexpr int SK_MAX_M = 8;

DEVINL void mma_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(SK_THREADS)
skinny_gemm_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ w, int M, int N, int K,
                   int ldx, int ldw, int ldo) {
    __shared__ float red[SK_WARPS][4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * SK_COLS;
    const bf16* w0 = w + (size_t)min(n0 + g, N - 1) * ldw;          // a clamped row is computed, not stored
    const bf16* w1 = w + (size_t)min(n0 + g + 8, N - 1) * ldw;
    const bool xvalid = g < M;
    const bf16* xr = x + (size_t)min(g, M - 1) * ldx;
    const int nchunks = (K + 31) >> 5;                               // 32 K elements per chunk: 8 per lane of a quad
    const int per_warp = (nchunks + SK_WARPS - 1) / SK_WARPS;
    const int c_begin = warp * per_warp, c_end = min(c_begin + per_warp, nchunks);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // whole groups of SK_UNROLL full chunks: every load is issued before the first MMA, nothing is predicated
    const int full_end = min(c_end, K >> 5);
    int ch = c_begin;
    for (; ch + SK_UNROLL <= full_end; ch += SK_UNROLL) {
        uint4 a0[SK_UNROLL], a1[SK_UNROLL], b[SK_UNROLL];
        #pragma unroll
        for (int u = 0; u < SK_UNROLL; u++) {
            const int k = ((ch + u) << 5) + t * 8;
            a0[u] = __ldcs(reinterpret_cast<const uint4*>(w0 + k));
            a1[u] = __ldcs(reinterpret_cast<const uint4*>(w1 + k));
            b[u] = *reinterpret_cast<const uint4*>(xr + k);
        }
        #pragma unroll
        for (int u = 0; u < SK_UNROLL; u++) {
            if (!xvalid) b[u] = zero;
            mma_16x8x16(c, a0[u].x, a1[u].x, a0[u].y, a1[u].y, b[u].x, b[u].y);
            mma_16x8x16(c, a0[u].z, a1[u].z, a0[u].w, a1[u].w, b[u].z, b[u].w);
        }
    }
    // the rest, one chunk at a time; the last chunk of K may be partial
    for (; ch < c_end; ch++) {
        const int k = (ch << 5) + t * 8;
        const bool ok = k < K;
        const uint4 a0 = ok ? __ldcs(reinterpret_cast<const uint4*>(w0 + k)) : zero;
        const uint4 a1 = ok ? __ldcs(reinterpret_cast<const uint4*>(w1 + k)) : zero;
        const uint4 b = (ok && xvalid) ? *reinterpret_cast<const uint4*>(xr + k) : zero;
        mma_16x8x16(c, a0.x, a1.x, a0.y, a1.y, b.x, b.y);
        mma_16x8x16(c, a0.z, a1.z, a0.w, a1.w, b.z, b.w);
    }
    #pragma unroll
    for (int i = 0; i < 4; i++) red[warp][i][lane] = c[i];
    __syncthreads();
    if (warp == 0) {
        // accumulator layout: c[2 i + j] = out[row 2 t + j][column n0 + g + 8 i]
        #pragma unroll
        for (int i = 0; i < 4; i++) {
            float v = 0.f;
            #pragma unroll
            for (int ww = 0; ww < SK_WARPS; ww++) v += red[ww][i][lane];
            const int m = 2 * t + (i & 1), n = n0 + g + 8 * (i >> 1);
            if (m < M && n < N) out[(size_t)m * ldo + n] = __float2bfloat16_rn(v);
        }
    }
}

int decode_check(int B, int Tq, int Tmax, int start_pos, int NH, int NKV, int HS, bool device_pos) {
    if (HS % 8 || HS > DEC_MAX_HS || HS < 16 || NKV <= 0 || NH % NKV) return -1;
    if (B <= 0 || Tq <= 0 || Tq > Tmax) return -2;
    if (!device_pos && (start_pos < 0 || start_pos + Tq > Tmax)) return -2;
    if (B > 65535 || Tq > 65535) return -3;
    return 0;
}

}  // namespace

// freqs holds (cos, sin) for freqs_len positions; every position written must lie inside it and inside the cache.
// pos_ptr: null, or a device int that replaces start_pos when the kernel runs.
extern "C" int llmc_rope_cache(bf16* q, bf16* kcache, bf16* vcache, const bf16* raw, const float* freqs, int freqs_len, int B, int Tq,
                               int Tmax, int start_pos, int NH, int NKV, int HS, const int* pos_ptr, cudaStream_t stream) {
    const int rc = decode_check(B, Tq, Tmax, start_pos, NH, NKV, HS, pos_ptr != nullptr);
    if (rc) return rc;
    if (!pos_ptr && start_pos + Tq > freqs_len) return -4;
    const long long N = (long long)B * Tq;
    const long long total = N * (NH + 2 * NKV) * (HS / 8);
    rope_cache_kernel<<<(unsigned)CEIL_DIV(total, 256), 256, 0, stream>>>(q, kcache, vcache, raw, reinterpret_cast<const float2*>(freqs),
                                                                          N, Tq, Tmax, start_pos, NH, NKV, HS, pos_ptr, freqs_len,
                                                                          llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

namespace {
// Key slices of the fast path: whole multiples of the 128 keys a CTA covers per trip, at least CA_MIN_KEYS, and short enough
// for about sixteen CTAs per SM (three are resident at a time: many short CTAs keep the last wave small).  The cache's
// capacity decides, not the current length, because the position may live on the device.
int ca_keys_per_slice(int B, int Tmax, int NKV) {
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int want = CEIL_DIV(16 * sms, B * NKV);
    int kps = CEIL_DIV(CEIL_DIV(Tmax, want), CA_WARPS * 32) * (CA_WARPS * 32);
    return kps < CA_MIN_KEYS ? CA_MIN_KEYS : kps;
}
int ca_slices(int B, int Tmax, int NKV) { return CEIL_DIV(Tmax, ca_keys_per_slice(B, Tmax, NKV)); }
int ca_rows_padded(int rows) { return rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8; }
bool ca_fast(int Tq, int NH, int NKV, int HS) { return (HS == 64 || HS == 128) && (NH / NKV) * Tq <= CA_MAX_R; }

template <int HS_, int R>
int ca_launch(bf16* out, float* ws, const bf16* q, const bf16* kcache, const bf16* vcache, int B, int Tq, int Tmax, int start_pos, int NH,
              int NKV, const int* pos_ptr, cudaStream_t stream) {
    const int rows = (NH / NKV) * Tq, slices = ca_slices(B, Tmax, NKV);
    const int keys_per_slice = ca_keys_per_slice(B, Tmax, NKV);
    constexpr int smem = ca_smem_bytes<HS_, R>();
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(cached_attention_split_kernel<HS_, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    cached_attention_split_kernel<HS_, R><<<dim3(slices, NKV, B), CA_THREADS, smem, stream>>>(ws, q, kcache, vcache, Tq, Tmax, start_pos, NH, NKV,
                                                                                           rsqrtf((float)HS_), pos_ptr, llmc_status_ptr(),
                                                                                           keys_per_slice, rows);
    CUDA_CHECK(cudaGetLastError());
    cached_attention_combine_kernel<HS_><<<dim3(rows, NKV, B), HS_, 0, stream>>>(out, ws, Tq, NH, NKV, slices, R, rows);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
}  // namespace

// fp32 words of workspace llmc_cached_attention needs for this problem (0: the general kernel runs, which needs none)
extern "C" long long llmc_cached_attention_workspace(int B, int Tq, int Tmax, int NH, int NKV, int HS) {
    if (NKV <= 0 || NH % NKV || !ca_fast(Tq, NH, NKV, HS)) return 0;
    return (long long)B * NKV * ca_slices(B, Tmax, NKV) * ca_rows_padded((NH / NKV) * Tq) * (HS + 2);
}

extern "C" int llmc_cached_attention(bf16* out, const bf16* q, const bf16* kcache, const bf16* vcache, int B, int Tq, int Tmax,
                                     int start_pos, int NH, int NKV, int HS, const int* pos_ptr, float* ws, cudaStream_t stream) {
    const int rc = decode_check(B, Tq, Tmax, start_pos, NH, NKV, HS, pos_ptr != nullptr);
    if (rc) return rc;
    if (ws != nullptr && ca_fast(Tq, NH, NKV, HS)) {
        if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache)) & 15) return -5;
        const int R = ca_rows_padded((NH / NKV) * Tq);
#define CA_GO(H, RR) return ca_launch<H, RR>(out, ws, q, kcache, vcache, B, Tq, Tmax, start_pos, NH, NKV, pos_ptr, stream)
        if (HS == 64) { if (R == 1) CA_GO(64, 1); if (R == 2) CA_GO(64, 2); if (R == 4) CA_GO(64, 4); CA_GO(64, 8); }
        else { if (R == 1) CA_GO(128, 1); if (R == 2) CA_GO(128, 2); if (R == 4) CA_GO(128, 4); CA_GO(128, 8); }
#undef CA_GO
    }
    const dim3 grid(NH, Tq, B);
    cached_attention_kernel<<<grid, DEC_THREADS, 0, stream>>>(out, q, kcache, vcache, Tq, Tmax, start_pos, NH, NKV, HS, rsqrtf((float)HS),
                                                              pos_ptr, llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// out (M, N) = x (M, K) . w (N, K)^T for M <= 8; K and the row strides of x and w are multiples of 8 elements.
extern "C" int llmc_skinny_gemm(bf16* out, const bf16* x, const bf16* w, int M, int N, int K, int ldx, int ldw, int ldo, cudaStream_t stream) {
    if (M <= 0 || M > SK_MAX_M || N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8)) return -1;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -1;
    skinny_gemm_kernel<<<(unsigned)CEIL_DIV(N, SK_COLS), SK_THREADS, 0, stream>>>(out, x, w, M, N, K, ldx, ldw, ldo);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
