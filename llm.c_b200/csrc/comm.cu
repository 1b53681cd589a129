// ZeRO-1 communication inside kernels, over NVLink peer memory (no NCCL call on these paths).
//
// Every rank holds pointers to all ranks' gradient buffer, parameter buffer and signal buffer
// (symmetric allocations, same layout everywhere).  Synchronisation uses 64-bit flags in the signal
// buffers that only ever grow (the step sequence number), written with st.release.sys after a
// system-scope fence and polled with ld.acquire.sys; every poll is bounded (FLAG_WAIT_CYCLES) and on
// expiry the kernel records ST_FLAG_TIMEOUT in the status word, skips its work and returns.
//
//  reduce_scatter   (per layer, on a side stream while backward continues)  signal "my gradients of
//                   channel c are final" to all peers, wait for theirs, then for each tensor of the layer
//                   read this rank's 1/N shard from every peer (plain peer loads, summed in rank order in
//                   fp32: deterministic and identical to a reduce with a fixed tree), scale by 1/N, store
//                   the bf16 mean into the own buffer's shard, and emit per-CTA partial sums of squares
//                   of the reduced values (the global gradient norm needs no second pass).
//                   Replaces ncclReduceScatter(ncclAvg) + global_norm_squared of the reference
//                   (llmc/zero.cuh:539-548, train_gpt2.cu:1002-1023).
//  all_reduce       the same kernel in its data-parallel (-z 0) form: the owner of a shard also stores the mean into every
//                   peer's gradient buffer and, when its last CTA is done, raises a "broadcast done" flag on every peer;
//                   the optimizer waits for all peers' flags.  Replaces ncclAllReduce(ncclAvg) (llmc/zero.cuh:532-538).
//  scalar all-reduce one-shot: every rank stores {sequence, value} as one 64-bit word into its slot of
//                   every peer's signal buffer and sums the N slots in rank order.
//  adamw_allgather  AdamW + stochastic rounding on the own shards; each rounded bf16 pack is stored to
//                   the own parameter buffer and to every peer's (16-byte peer stores), the last CTA to
//                   finish raises this rank's "parameters published" flag of the launch's channel on all
//                   peers.  The caller launches it once per parameter group in the order the forward pass
//                   consumes the groups; the consumer is the first GEMM that reads a group's weights (its
//                   TMA producer polls the group's flags before its first load, see gemm2.cu), so the forward
//                   pass of early layers runs while later groups are still being updated and gathered.
//                   Replaces adamw_kernel3 + ncclAllGather (train_gpt2.cu:1101-1120 of the reference).
//  wait_flags       tiny kernel for consumers that are not GEMMs (embedding lookup, checkpoint writer).
#include "common.cuh"

struct TensorView {        // same layout as in optim.cu
    long long p_base, p_stride, o_base, o_stride, n;
    int L;
    float wd;
    unsigned int seed;
    int pad;
};
struct TensorTable {
    TensorView t[16];
    int count;
};

constexpr int MAX_RANKS = 8;       // one NVSwitch domain
struct PeerPtrs {
    void* p[MAX_RANKS];
};
struct SliceList {
    long long off[16];
    long long size[16];
    int count;
};

#ifndef FLAG_WAIT_CYCLES
#define FLAG_WAIT_CYCLES (20000000000ll)      // roughly 10 s
#endif

// signal buffer layout (64-bit words)
constexpr int SIG_RS_BASE = 0;          // [channel 0..199][src rank]  "my gradients of this group are final"
constexpr int SIG_AG_BASE = 200 * MAX_RANKS;    // [channel 0..199][src rank]  "parameters of this group are published"
constexpr int SIG_AR_BASE = 400 * MAX_RANKS;    // [channel 0..199][src rank]  "my shard of this group's mean gradient is in your buffer"
constexpr int SIG_BARRIER = 600 * MAX_RANKS;
constexpr int SIG_SCALAR = 601 * MAX_RANKS;     // [parity][value 0..3][src rank] packed {seq, float}
constexpr int MAX_SCALARS = 4;
constexpr int SIG_WORDS = (601 + 2 * MAX_SCALARS) * MAX_RANKS;
constexpr int MAX_CHANNELS = 200;

// limit of every peer-flag wait in clock cycles; adjustable at run time (tests shorten it)
__device__ long long g_flag_wait_cycles = FLAG_WAIT_CYCLES;

namespace {

DEVINL void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
DEVINL unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// wait until *p >= want; false on time-out
DEVINL bool wait_flag_ge(const unsigned long long* p, unsigned long long want, unsigned int* status, unsigned int where) {
    long long t0 = clock64();
    while (ld_acquire_sys(p) < want) {
        if (clock64() - t0 > g_flag_wait_cycles) { record_error(status, ST_FLAG_TIMEOUT, where); return false; }
        __nanosleep(200);
    }
    return true;
}

// Two shapes of CTA.  The default is 512 threads: such a CTA takes a whole SM (the backward kernels running on the main stream are
// persistent CTAs that fill an SM's shared memory and most of its registers), so 32 of them keep the reduce-scatter on 32 SMs.
// The alternative, 128 threads with 48 registers and no shared memory, fits next to the compute CTAs on every SM; measured on two
// GPUs with one micro-step per step it was 1.3 % slower end to end (74.4 against 73.4 ms), so it is only kept selectable.
constexpr int RS_THREADS = 128;

// U packs of 8 elements per thread and trip, from up to NMAX ranks each: U * NMAX = 8 independent 16-byte loads are in flight per
// thread whatever the number of ranks (NVLink latency is what this loop hides; with two ranks and one pack per trip the link
// ran at a quarter of its rate).
template <int THREADS, int U, int NMAX>
__global__ void __launch_bounds__(THREADS, THREADS == RS_THREADS ? 10 : 1)
reduce_scatter_kernel(PeerPtrs grads, PeerPtrs sig, SliceList sl, int rank, int N, float scale, int channel,
                      unsigned long long seq, float* __restrict__ norm_partials, int wait_peers, int allreduce,
                      unsigned int* __restrict__ done_counter, unsigned int* status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long* my_sig = reinterpret_cast<unsigned long long*>(sig.p[rank]);
    // wait_peers == 2: the exchange of "gradients final" flags already happened in rs_handshake_kernel, launched before this
    // kernel, so that no SM is held while the slowest peer is still computing.
    // 1. tell every peer that this rank's gradients of `channel` are final (one warp of block 0)
    if (wait_peers != 2 && blockIdx.x == 0 && threadIdx.x < N) {
        __threadfence_system();
        unsigned long long* peer = reinterpret_cast<unsigned long long*>(sig.p[threadIdx.x]);
        st_release_sys(peer + SIG_RS_BASE + channel * MAX_RANKS + rank, seq);
    }
    // 2. the first warp waits for every peer's signal (lane p polls peer p; few pollers: every poll is a system-scope load that
    //    goes to L2); the verdict reaches the other warps through the barrier itself, so no shared memory is needed
    bool ok = true;
    if (wait_peers == 1) {
        bool mine_ok = true;
        if (warp == 0 && lane < N) mine_ok = wait_flag_ge(my_sig + SIG_RS_BASE + channel * MAX_RANKS + lane, seq, status, 0x700 + lane);
        ok = __syncthreads_and(mine_ok) != 0;
    }
    float acc_sq = 0.f;
    if (ok) {
        bf16* mine = reinterpret_cast<bf16*>(grads.p[rank]);
        for (int s = 0; s < sl.count; s++) {
            const long long shard = sl.size[s] / N;
            const long long base = sl.off[s] + (long long)rank * shard;
            const long long packs = shard >> 3;
            for (long long i0 = (long long)blockIdx.x * (THREADS * U) + threadIdx.x; i0 < packs; i0 += (long long)gridDim.x * (THREADS * U)) {
                float sum[U][8];
                #pragma unroll
                for (int u = 0; u < U; u++)
                    #pragma unroll
                    for (int e = 0; e < 8; e++) sum[u][e] = 0.f;
                // rank order: the same sum on every run.  The small CTAs have the registers for four vectors at a time.
                constexpr int GROUP = THREADS == RS_THREADS ? 4 : NMAX;
                #pragma unroll
                for (int p0 = 0; p0 < NMAX; p0 += GROUP) {
                    if (p0 < N) {
                        bf16x8 v[U][GROUP];
                        #pragma unroll
                        for (int u = 0; u < U; u++)
                            #pragma unroll
                            for (int k = 0; k < GROUP; k++)
                                if (p0 + k < N && i0 + u * THREADS < packs)
                                    v[u][k] = ld128cs(reinterpret_cast<const bf16*>(grads.p[p0 + k]) + base + (i0 + u * THREADS) * 8);
                        #pragma unroll
                        for (int u = 0; u < U; u++)
                            #pragma unroll
                            for (int k = 0; k < GROUP; k++) {
                                if (p0 + k < N && i0 + u * THREADS < packs) {
                                    #pragma unroll
                                    for (int e = 0; e < 8; e++) sum[u][e] += __bfloat162float(v[u][k][e]);
                                }
                            }
                    }
                }
                #pragma unroll
                for (int u = 0; u < U; u++) {
                    const long long i = i0 + u * THREADS;
                    if (i < packs) {
                        bf16x8 o;
                        #pragma unroll
                        for (int e = 0; e < 8; e++) {
                            o[e] = __float2bfloat16_rn(sum[u][e] * scale);
                            const float f = __bfloat162float(o[e]);
                            acc_sq += f * f;
                        }
                        if (allreduce) {
                            #pragma unroll
                            for (int p = 0; p < NMAX; p++)
                                if (p < N) st128(reinterpret_cast<bf16*>(grads.p[p]) + base + i * 8, o);      // own copy and every peer's
                        } else {
                            st128(mine + base + i * 8, o);
                        }
                    }
                }
            }
        }
    }
    // one partial sum of squares per warp (the host adds them all)
    acc_sq = warp_sum(acc_sq);
    if (lane == 0 && norm_partials) norm_partials[blockIdx.x * (THREADS / 32) + warp] = acc_sq;
    if (allreduce) {
        // the last CTA to get here tells every peer that this rank's shard of the channel has landed in its buffer
        __threadfence_system();
        const int last = __syncthreads_or(threadIdx.x == 0 && atomicAdd(done_counter, 1u) == gridDim.x - 1);
        if (last) {
            if (threadIdx.x == 0) *done_counter = 0;
            if (threadIdx.x < N) {
                __threadfence_system();
                unsigned long long* peer = reinterpret_cast<unsigned long long*>(sig.p[threadIdx.x]);
                st_release_sys(peer + SIG_AR_BASE + channel * MAX_RANKS + rank, seq);
            }
        }
    }
}

// inout[v] = sum over ranks of inout[v], v < count <= MAX_SCALARS, summed in rank order (the same bits on every rank).  Before
// the exchange, inout[0] may be replaced by the sum of `n_partials` partial sums (the squared-norm partials of the
// reduce-scatter launches) and inout[1] by scale1 * sum of `n_terms` terms (the per-token losses): both sums use a fixed
// tree, so the training loop needs no library reduction between backward and the update.
__global__ void __launch_bounds__(256)
scalar_allreduce_kernel(PeerPtrs sig, float* __restrict__ inout, int count, const float* __restrict__ partials, int n_partials,
                        const float* __restrict__ terms, int n_terms, float scale1, int rank, int N, unsigned long long seq,
                        unsigned int* status) {
    __shared__ float red[32];
    __shared__ float vals[MAX_SCALARS][MAX_RANKS];
    __shared__ int ok_s;
    if (partials != nullptr) {
        float acc = 0.f;
        for (int i = threadIdx.x; i < n_partials; i += blockDim.x) acc += partials[i];
        acc = block_sum(acc, red);
        if (threadIdx.x == 0) inout[0] = acc;
    }
    if (terms != nullptr) {
        float acc = 0.f;
        for (int i = threadIdx.x; i < n_terms; i += blockDim.x) acc += terms[i];
        acc = block_sum(acc, red);
        if (threadIdx.x == 0) inout[1] = acc * scale1;
    }
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (N == 1) return;
    unsigned long long* my_sig = reinterpret_cast<unsigned long long*>(sig.p[rank]);
    const int parity = (int)(seq & 1);
    const int v = threadIdx.x / MAX_RANKS, p = threadIdx.x % MAX_RANKS;
    if (v < count && p < N) {
        const unsigned long long word = (seq << 32) | (unsigned long long)__float_as_uint(inout[v]);
        unsigned long long* peer = reinterpret_cast<unsigned long long*>(sig.p[p]);
        st_release_sys(peer + SIG_SCALAR + (parity * MAX_SCALARS + v) * MAX_RANKS + rank, word);
        // wait for slot (v, p) of my own buffer to carry this sequence number
        const unsigned long long* slot = my_sig + SIG_SCALAR + (parity * MAX_SCALARS + v) * MAX_RANKS + p;
        long long t0 = clock64();
        unsigned long long w;
        while (((w = ld_acquire_sys(slot)) >> 32) < (seq & 0xFFFFFFFFull)) {
            if (clock64() - t0 > g_flag_wait_cycles) { record_error(status, ST_FLAG_TIMEOUT, 0x720 + p); ok_s = 0; break; }
            __nanosleep(100);
        }
        vals[v][p] = __uint_as_float((unsigned int)(w & 0xFFFFFFFFull));
    }
    __syncthreads();
    if (threadIdx.x < count && ok_s) {
        float s = 0.f;
        for (int q = 0; q < N; q++) s += vals[threadIdx.x][q];
        inout[threadIdx.x] = s;
    }
}

DEVINL unsigned int sr_position(long long idx, int layer) {
    return (unsigned int)(idx & 511) + 198491317u * ((unsigned int)(idx & ~511ll) + (unsigned int)layer);
}

template <bool HAS_MASTER>
__global__ void __launch_bounds__(512)
adamw_allgather_kernel(PeerPtrs params, PeerPtrs sig, float* __restrict__ master, const bf16* __restrict__ grads,
                       float* __restrict__ m_buf, float* __restrict__ v_buf, const TensorTable tab, int rank, int N,
                       float lr, float beta1, float beta2, float bc1, float bc2, float eps, float grad_scale,
                       const float* __restrict__ norm_sq, float grad_clip, unsigned long long seq,
                       unsigned int* __restrict__ done_counter, int channel) {
    float scale = grad_scale;
    bool skip = false;
    if (norm_sq != nullptr) {
        const float nsq = norm_sq[0];
        if (!(nsq >= 0.f) || isinf(nsq)) skip = true;      // non-finite gradient: publish the unchanged parameters
        else { const float nrm = sqrtf(nsq); if (nrm > grad_clip) scale = grad_scale * grad_clip / nrm; }
    }
    bf16* mine = reinterpret_cast<bf16*>(params.p[rank]);
    for (int ti = 0; ti < tab.count; ti++) {
        const TensorView tv = tab.t[ti];
        const long long packs_per_slice = tv.n >> 3;
        const long long total = packs_per_slice * tv.L;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
            const long long l = i / packs_per_slice, pk = i - l * packs_per_slice;
            const long long pi = tv.p_base + l * tv.p_stride + pk * 8;
            const long long oi = tv.o_base + l * tv.o_stride + pk * 8;
            bf16x8 out;
            if (!skip) {
                const bf16x8 g = ld128cs(grads + pi);
                f32x4 m0 = ld128(m_buf + oi), m1 = ld128(m_buf + oi + 4), v0 = ld128(v_buf + oi), v1 = ld128(v_buf + oi + 4);
                f32x4 w0, w1;
                if (HAS_MASTER) { w0 = ld128(master + oi); w1 = ld128(master + oi + 4); }
                else { bf16x8 pw = ld128(mine + pi);
                       #pragma unroll
                       for (int e = 0; e < 4; e++) { w0[e] = __bfloat162float(pw[e]); w1[e] = __bfloat162float(pw[e + 4]); } }
                #pragma unroll
                for (int e = 0; e < 8; e++) {
                    float& mm = e < 4 ? m0[e] : m1[e - 4];
                    float& vv = e < 4 ? v0[e] : v1[e - 4];
                    float& ww = e < 4 ? w0[e] : w1[e - 4];
                    const float gg = scale * __bfloat162float(g[e]);
                    mm = fmaf(beta1, mm, (1.0f - beta1) * gg);
                    vv = fmaf(beta2, vv, (1.0f - beta2) * gg * gg);
                    const float mh = mm / bc1, vh = vv / bc2;
                    ww = ww - lr * (mh / (sqrtf(vh) + eps) + tv.wd * ww);
                    out[e] = stochastic_round_bf16(ww, squirrel_noise5(sr_position(pk * 8 + e, (int)l + tv.pad), tv.seed));
                }
                st128(m_buf + oi, m0); st128(m_buf + oi + 4, m1); st128(v_buf + oi, v0); st128(v_buf + oi + 4, v1);
                if (HAS_MASTER) { st128(master + oi, w0); st128(master + oi + 4, w1); }
            } else {
                out = ld128(mine + pi);
            }
            #pragma unroll
            for (int p = 0; p < MAX_RANKS; p++)
                if (p < N) st128(reinterpret_cast<bf16*>(params.p[p]) + pi, out);      // own copy and every peer's
        }
    }
    // publish: the last CTA to get here raises this rank's flag on every peer
    __threadfence_system();
    __syncthreads();
    __shared__ int last;
    if (threadIdx.x == 0) {
        unsigned int prev = atomicAdd(done_counter, 1u);
        last = (prev == gridDim.x - 1);
        if (last) *done_counter = 0;
    }
    __syncthreads();
    if (last && threadIdx.x < N) {
        __threadfence_system();
        unsigned long long* peer = reinterpret_cast<unsigned long long*>(sig.p[threadIdx.x]);
        st_release_sys(peer + SIG_AG_BASE + channel * MAX_RANKS + rank, seq);
    }
}

// waits for the N flags of each of `nch` consecutive channels starting at word `base`
__global__ void wait_flags_kernel(PeerPtrs sig, int rank, int N, int base, int nch, unsigned long long seq, unsigned int* status) {
    const unsigned long long* my_sig = reinterpret_cast<const unsigned long long*>(sig.p[rank]);
    const int p = threadIdx.x % MAX_RANKS;
    if (p < N)
        for (int ch = threadIdx.x / MAX_RANKS; ch < nch; ch += blockDim.x / MAX_RANKS)
            if (!wait_flag_ge(my_sig + base + ch * MAX_RANKS + p, seq, status, 0x740 + p)) break;
}

// One warp: tells every peer that this rank's gradients of `channel` are final and waits until every peer has said the same.
// It runs ahead of the wide reduction on the communication stream; while it waits it occupies one warp slot, not 32 SMs.
__global__ void __launch_bounds__(32) rs_handshake_kernel(PeerPtrs sig, int rank, int N, int channel, unsigned long long seq, unsigned int* status) {
    const int lane = threadIdx.x;
    if (lane < N) {
        __threadfence_system();
        unsigned long long* peer = reinterpret_cast<unsigned long long*>(sig.p[lane]);
        st_release_sys(peer + SIG_RS_BASE + channel * MAX_RANKS + rank, seq);
        const unsigned long long* my_sig = reinterpret_cast<const unsigned long long*>(sig.p[rank]);
        wait_flag_ge(my_sig + SIG_RS_BASE + channel * MAX_RANKS + lane, seq, status, 0x720 + lane);
    }
}

__global__ void signal_flags_kernel(PeerPtrs sig, int rank, int N, int base, unsigned long long seq) {
    if (threadIdx.x < N) {
        __threadfence_system();
        unsigned long long* peer = reinterpret_cast<unsigned long long*>(sig.p[threadIdx.x]);
        st_release_sys(peer + base + rank, seq);
    }
}

int fill(PeerPtrs* pp, const unsigned long long* ptrs, int N) {
    if (N < 1 || N > MAX_RANKS) return -1;
    for (int i = 0; i < MAX_RANKS; i++) pp->p[i] = i < N ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
    return 0;
}

}  // namespace

extern "C" int llmc_p2p_signal_words() { return SIG_WORDS; }

// Sets the limit (clock cycles) after which a wait on a peer flag gives up and records ST_FLAG_TIMEOUT. 0 restores the default.
static long long h_flag_wait_cycles = FLAG_WAIT_CYCLES;      // host mirror, for kernels of other files that take the limit as an argument
long long llmc_p2p_wait_cycles_host() { return h_flag_wait_cycles; }

extern "C" int llmc_p2p_set_wait_cycles(long long cycles) {
    long long v = cycles > 0 ? cycles : FLAG_WAIT_CYCLES;
    CUDA_CHECK(cudaMemcpyToSymbol(g_flag_wait_cycles, &v, sizeof(v)));
    h_flag_wait_cycles = v;
    return 0;
}

// LLMC_RS_THREADS=128 selects the small CTAs for the reduce-scatter (for measurements of the difference); the default is 512.
static int rs_threads() {
    static int v = 0;
    if (v == 0) { const char* e = getenv("LLMC_RS_THREADS"); v = (e && atoi(e) == RS_THREADS) ? RS_THREADS : 512; }
    return v;
}

// Reduce-scatter (mean) of up to 16 slices of the gradient buffers. grad_ptrs / sig_ptrs: N device pointers (one per rank).
// Every slice size must be a multiple of 8*N. norm_partials: llmc_p2p_rs_partials(ctas) floats (may be null).
// wait_peers: 1 = the reduction kernel itself exchanges the "gradients final" flags and waits; 2 = llmc_p2p_rs_handshake already
// did, in an earlier launch (the wide kernel then never spins); 0 = signal only (single-process tests).
extern "C" int llmc_p2p_reduce_scatter(const unsigned long long* grad_ptrs, const unsigned long long* sig_ptrs, const long long* offs,
                                       const long long* sizes, int count, int rank, int N, int channel, unsigned long long seq,
                                       float* norm_partials, int ctas, int wait_peers, int allreduce, unsigned int* done_counter,
                                       cudaStream_t stream) {
    PeerPtrs g, s; SliceList sl;
    if (fill(&g, grad_ptrs, N) || fill(&s, sig_ptrs, N) || count > 16 || channel < 0 || channel >= 200) return -1;
    if (allreduce && done_counter == nullptr) return -1;
    sl.count = count;
    for (int i = 0; i < count; i++) { sl.off[i] = offs[i]; sl.size[i] = sizes[i]; if (sizes[i] % (8 * N) || offs[i] % 8) return -2; }
#define RS_LAUNCH(T, U, NM) reduce_scatter_kernel<T, U, NM><<<ctas, T, 0, stream>>>(g, s, sl, rank, N, 1.0f / N, channel, seq, norm_partials, \
                                                                                    wait_peers, allreduce, done_counter, llmc_status_ptr())
    if (rs_threads() != 512) RS_LAUNCH(RS_THREADS, 1, 8);
    else if (N <= 2) RS_LAUNCH(512, 4, 2);
    else if (N <= 4) RS_LAUNCH(512, 2, 4);
    else RS_LAUNCH(512, 1, 8);
#undef RS_LAUNCH
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// The exchange of "gradients of `channel` are final" flags as a launch of its own (one warp).  A reduce-scatter launched with
// wait_peers = 2 after it, on this stream or on one that waits for it, finds every peer's gradients final.
extern "C" int llmc_p2p_rs_handshake(const unsigned long long* sig_ptrs, int rank, int N, int channel, unsigned long long seq,
                                     cudaStream_t stream) {
    PeerPtrs s;
    if (fill(&s, sig_ptrs, N) || channel < 0 || channel >= 200) return -1;
    rs_handshake_kernel<<<1, 32, 0, stream>>>(s, rank, N, channel, seq, llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// number of partial sums of squares a reduce-scatter launch of `ctas` CTAs writes
extern "C" int llmc_p2p_rs_partials(int ctas) { return ctas * (rs_threads() / 32); }

// Sum of `count` (<= 4) device floats over the ranks, in place.  Optional fused local sums first: inout[0] = sum(partials),
// inout[1] = scale1 * sum(terms).  A sequence number may be used once; consecutive calls use consecutive numbers.
extern "C" int llmc_p2p_allreduce_scalars(const unsigned long long* sig_ptrs, float* inout, int count, const float* partials, int n_partials,
                                          const float* terms, int n_terms, float scale1, int rank, int N, unsigned long long seq,
                                          cudaStream_t stream) {
    PeerPtrs s;
    if (fill(&s, sig_ptrs, N) || count < 1 || count > MAX_SCALARS || (terms && count < 2)) return -1;
    scalar_allreduce_kernel<<<1, 256, 0, stream>>>(s, inout, count, partials, n_partials, terms, n_terms, scale1, rank, N, seq, llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_p2p_allreduce_scalar(const unsigned long long* sig_ptrs, float* inout, int rank, int N, unsigned long long seq,
                                         cudaStream_t stream) {
    return llmc_p2p_allreduce_scalars(sig_ptrs, inout, 1, nullptr, 0, nullptr, 0, 1.0f, rank, N, seq, stream);
}

extern "C" int llmc_p2p_adamw_allgather(const unsigned long long* param_ptrs, const unsigned long long* sig_ptrs, float* master,
                                        const bf16* grads, float* m, float* v, const TensorTable* tab, int rank, int N,
                                        float lr, float beta1, float beta2, float eps, int t, float grad_scale, const float* norm_sq,
                                        float grad_clip, unsigned long long seq, unsigned int* done_counter, int ctas, int channel,
                                        cudaStream_t stream) {
    PeerPtrs p, s;
    if (fill(&p, param_ptrs, N) || fill(&s, sig_ptrs, N)) return -1;
    if (channel < 0 || channel >= MAX_CHANNELS) return -3;
    for (int i = 0; i < tab->count; i++) if (tab->t[i].n % 8 || tab->t[i].p_base % 8 || tab->t[i].p_stride % 8 || tab->t[i].o_base % 8 || tab->t[i].o_stride % 8) return -2;
    const float bc1 = 1.0f - powf(beta1, (float)t), bc2 = 1.0f - powf(beta2, (float)t);
    if (master) adamw_allgather_kernel<true><<<ctas, 512, 0, stream>>>(p, s, master, grads, m, v, *tab, rank, N, lr, beta1, beta2, bc1, bc2, eps, grad_scale, norm_sq, grad_clip, seq, done_counter, channel);
    else adamw_allgather_kernel<false><<<ctas, 512, 0, stream>>>(p, s, master, grads, m, v, *tab, rank, N, lr, beta1, beta2, bc1, bc2, eps, grad_scale, norm_sq, grad_clip, seq, done_counter, channel);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// word offset, inside a rank's signal buffer, of the N "published" flags of a parameter group
extern "C" int llmc_p2p_ag_flag_offset(int channel) { return SIG_AG_BASE + channel * MAX_RANKS; }

// which: 0 = parameters of `channel` published (all-gather), 1 = barrier, 2 = mean gradients of `channel` broadcast (all-reduce)
extern "C" int llmc_p2p_wait(const unsigned long long* sig_ptrs, int rank, int N, int which, int channel, unsigned long long seq,
                             cudaStream_t stream) {
    PeerPtrs s;
    if (fill(&s, sig_ptrs, N)) return -1;
    if (which != 1 && (channel < 0 || channel >= MAX_CHANNELS)) return -3;
    const int base = which == 0 ? SIG_AG_BASE + channel * MAX_RANKS : which == 2 ? SIG_AR_BASE + channel * MAX_RANKS : SIG_BARRIER;
    wait_flags_kernel<<<1, 32, 0, stream>>>(s, rank, N, base, 1, seq, llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// the same for `nch` consecutive channels in one launch (which: 0 or 2)
extern "C" int llmc_p2p_wait_range(const unsigned long long* sig_ptrs, int rank, int N, int which, int channel0, int nch, unsigned long long seq,
                                   cudaStream_t stream) {
    PeerPtrs s;
    if (fill(&s, sig_ptrs, N)) return -1;
    if ((which != 0 && which != 2) || channel0 < 0 || nch < 1 || channel0 + nch > MAX_CHANNELS) return -3;
    const int base = (which == 0 ? SIG_AG_BASE : SIG_AR_BASE) + channel0 * MAX_RANKS;
    wait_flags_kernel<<<1, 256, 0, stream>>>(s, rank, N, base, nch, seq, llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// Device-side barrier across ranks on `stream`: signal, then wait for everyone.
extern "C" int llmc_p2p_barrier(const unsigned long long* sig_ptrs, int rank, int N, unsigned long long seq, cudaStream_t stream) {
    PeerPtrs s;
    if (fill(&s, sig_ptrs, N)) return -1;
    signal_flags_kernel<<<1, 32, 0, stream>>>(s, rank, N, SIG_BARRIER, seq);
    CUDA_CHECK(cudaGetLastError());
    wait_flags_kernel<<<1, 32, 0, stream>>>(s, rank, N, SIG_BARRIER, 1, seq, llmc_status_ptr());
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
