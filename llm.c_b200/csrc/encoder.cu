// Token + position embedding forward and its deterministic backward.
//
// Backward for the token table is a scatter-add with many collisions.  The reference builds
// buckets on the CPU every micro-step (llmc/encoder.cuh:187-228), stalling the GPU.  Here the
// bucketing happens on the device inside the same kernel: each CTA owns 64 consecutive token ids,
// scans the (L2-resident) token array in position order, compacts the positions that hit its range
// into shared memory (which therefore come out sorted by position), and then each warp adds up the
// rows of "its" ids in that fixed order.  One writer per table row, fixed summation order: the
// result is bit-reproducible and needs no atomics, no sort and no host work.
//
// Capability parity: llmc/encoder.cuh (encoder_forward, encoder_backward) of the reference.
#include "common.cuh"

namespace {

__global__ void encoder_fwd_kernel(bf16* __restrict__ out, const int* __restrict__ tokens, const bf16* __restrict__ wte,
                                   const bf16* __restrict__ wpe, int B, int T, int C, int V) {
    const int cp = C >> 3;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * T * cp) return;
    const int p = (int)(idx % cp);
    const long long bt = idx / cp;
    const int t = (int)(bt % T);
    (void)LLMC_DBG_CHECK(tokens[bt] >= 0 && tokens[bt] < V, 0xE01);     // debug build: an id outside the table is reported
    const int tok = min(max(tokens[bt], 0), V - 1);      // ids are validated on the host; never index outside the table
    bf16x8 a = ld128(wte + (size_t)tok * C + p * 8);
    if (wpe == nullptr) {                                // models with rotary positions have no position table
        st128cs(out + bt * C + p * 8, a);
        return;
    }
    bf16x8 b = ld128(wpe + (size_t)t * C + p * 8);
    bf16x8 o;
    #pragma unroll
    for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(__bfloat162float(a[e]) + __bfloat162float(b[e]));
    st128cs(out + bt * C + p * 8, o);
}

// dwpe[t, c] (+)= sum_b dout[b, t, c]
__global__ void wpe_bwd_kernel(bf16* __restrict__ dwpe, const bf16* __restrict__ dout, int B, int T, int C,
                               int accumulate, unsigned int seed) {
    const int cp = C >> 3;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * cp) return;
    const int p = idx % cp, t = idx / cp;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int b = 0; b < B; b++) {
        bf16x8 d = ld128cs(dout + ((size_t)b * T + t) * C + p * 8);
        #pragma unroll
        for (int e = 0; e < 8; e++) acc[e] += __bfloat162float(d[e]);
    }
    bf16* dst = dwpe + (size_t)t * C + p * 8;
    bf16x8 o;
    if (accumulate) {
        bf16x8 old = ld128(dst);
        #pragma unroll
        for (int e = 0; e < 8; e++)
            o[e] = stochastic_round_bf16(acc[e] + __bfloat162float(old[e]), squirrel_noise5((unsigned)(idx * 8 + e), seed));
    } else {
        #pragma unroll
        for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(acc[e]);
    }
    st128(dst, o);
}

constexpr int IDS_PER_CTA = 64;
constexpr int LIST_CAP = 4096;
constexpr int WTE_THREADS = 256;
constexpr int WTE_MAXP = 8;     // channel packs per lane per pass => 2048 channels per pass
constexpr int WTE_SCAN = 4;     // sub-blocks of WTE_THREADS positions per scan round
static_assert(WTE_SCAN * (WTE_THREADS / 32) == 32, "the scan of the hit counts is one warp wide");

// dwte[v, :] (+)= sum over positions i (ascending) with tokens[i] == v of dout[i, :]
__global__ void __launch_bounds__(WTE_THREADS)
wte_bwd_kernel(bf16* __restrict__ dwte, const bf16* __restrict__ dout, const int* __restrict__ tokens,
               int N, int C, int V, int accumulate, unsigned int seed) {
    __shared__ int list_pos[LIST_CAP];
    __shared__ unsigned char list_id[LIST_CAP];
    __shared__ int warp_counts[WTE_SCAN * (WTE_THREADS / 32)];
    __shared__ int warp_base[WTE_SCAN * (WTE_THREADS / 32)];
    __shared__ int list_len;
    __shared__ int touched[IDS_PER_CTA];     // has this id already been written in this launch (multi-round case)

    const int v0 = blockIdx.x * IDS_PER_CTA;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = WTE_THREADS / 32;
    const int npack = C >> 3;
    if (threadIdx.x < IDS_PER_CTA) touched[threadIdx.x] = 0;
    if (threadIdx.x == 0) list_len = 0;
    __syncthreads();

    int pos0 = 0;
    while (pos0 < N) {
        // ---- scan: append matching positions in position order until the list is full.  A round covers WTE_SCAN sub-blocks of
        //      256 positions with ONE set of barriers: per (sub-block, warp) hit counts, an exclusive scan of the 32 counts by
        //      warp 0, then every hit is written at its final slot.  (One sub-block per round spent most of the kernel in its
        //      three barriers per 256 tokens.)
        while (pos0 < N) {
            if (list_len + WTE_SCAN * WTE_THREADS > LIST_CAP) break;      // uniform: list_len is read after a barrier
            int tok[WTE_SCAN];
            unsigned ballot[WTE_SCAN];
            #pragma unroll
            for (int k = 0; k < WTE_SCAN; k++) {
                const int i = pos0 + k * WTE_THREADS + threadIdx.x;
                tok[k] = (i < N) ? tokens[i] : -1;
                const bool hit = (tok[k] >= v0) && (tok[k] < v0 + IDS_PER_CTA);
                ballot[k] = __ballot_sync(0xffffffffu, hit);
                if (lane == 0) warp_counts[k * nwarps + warp] = __popc(ballot[k]);
            }
            __syncthreads();
            if (warp == 0) {                                   // WTE_SCAN * nwarps == 32 counts, in position order
                const int base0 = list_len;
                const int c = warp_counts[lane];
                int incl = c;
                #pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += t;
                }
                warp_base[lane] = base0 + incl - c;
                __syncwarp();
                if (lane == 31) list_len = base0 + incl;
            }
            __syncthreads();
            #pragma unroll
            for (int k = 0; k < WTE_SCAN; k++) {
                if ((ballot[k] >> lane) & 1u) {
                    const int slot = warp_base[k * nwarps + warp] + __popc(ballot[k] & ((1u << lane) - 1u));
                    list_pos[slot] = pos0 + k * WTE_THREADS + threadIdx.x;
                    list_id[slot] = (unsigned char)(tok[k] - v0);
                }
            }
            __syncthreads();                                   // the list is complete; the count tables may be rewritten
            pos0 += WTE_SCAN * WTE_THREADS;
        }
        const int len = list_len;
        // ---- reduce: warp w handles ids w, w + nwarps, ... ----
        for (int id = warp; id < IDS_PER_CTA; id += nwarps) {
            const int v = v0 + id;
            if (v >= V) break;
            for (int pbase = 0; pbase < npack; pbase += 32 * WTE_MAXP) {
                float acc[WTE_MAXP][8];
                #pragma unroll
                for (int i = 0; i < WTE_MAXP; i++)
                    #pragma unroll
                    for (int e = 0; e < 8; e++) acc[i][e] = 0.f;
                bool any = false;
                for (int l0 = 0; l0 < len; l0 += 32) {
                    const int l = l0 + lane;
                    const bool mine = (l < len) && (list_id[l] == id);
                    unsigned m = __ballot_sync(0xffffffffu, mine);
                    while (m) {
                        const int j = __ffs(m) - 1;
                        m &= m - 1;
                        any = true;
                        const bf16* src = dout + (size_t)list_pos[l0 + j] * C;
                        #pragma unroll
                        for (int i = 0; i < WTE_MAXP; i++) {
                            const int p = pbase + lane + 32 * i;
                            if (p < npack) {
                                bf16x8 d = ld128cs(src + p * 8);
                                #pragma unroll
                                for (int e = 0; e < 8; e++) acc[i][e] += __bfloat162float(d[e]);
                            }
                        }
                    }
                }
                const bool add_old = accumulate || touched[id];
                if (any || (!add_old)) {
                    bf16* dst = dwte + (size_t)v * C;
                    #pragma unroll
                    for (int i = 0; i < WTE_MAXP; i++) {
                        const int p = pbase + lane + 32 * i;
                        if (p < npack) {
                            bf16x8 o;
                            if (add_old) {
                                bf16x8 old = ld128(dst + p * 8);
                                #pragma unroll
                                for (int e = 0; e < 8; e++)
                                    o[e] = stochastic_round_bf16(acc[i][e] + __bfloat162float(old[e]),
                                                                 squirrel_noise5((unsigned)(v * C + p * 8 + e), seed));
                            } else {
                                #pragma unroll
                                for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(acc[i][e]);
                            }
                            st128(dst + p * 8, o);
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

}  // namespace

extern "C" int llmc_encoder_fwd(bf16* out, const int* tokens, const bf16* wte, const bf16* wpe, int B, int T, int C, int V, cudaStream_t stream) {
    if (C % 8) return -1;
    long long total = (long long)B * T * (C / 8);
    encoder_fwd_kernel<<<(unsigned)CEIL_DIV(total, 256), 256, 0, stream>>>(out, tokens, wte, wpe, B, T, C, V);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// accumulate_* = 0: the table is overwritten (rows of dwte without any hit become zero); 1: added to.
// (With tied embeddings dwte already holds the LM-head weight gradient, so it is normally added to.)
extern "C" int llmc_encoder_bwd(bf16* dwte, bf16* dwpe, const bf16* dout, const int* tokens, int B, int T, int C, int V,
                                int accumulate_wte, int accumulate_wpe, unsigned int seed, cudaStream_t stream) {
    if (C % 8) return -1;
    if (dwpe != nullptr) {
        wpe_bwd_kernel<<<CEIL_DIV(T * (C / 8), 256), 256, 0, stream>>>(dwpe, dout, B, T, C, accumulate_wpe, seed);
        CUDA_CHECK(cudaGetLastError());
    }
    wte_bwd_kernel<<<CEIL_DIV(V, IDS_PER_CTA), WTE_THREADS, 0, stream>>>(dwte, dout, tokens, B * T, C, V, accumulate_wte, seed + 1);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
