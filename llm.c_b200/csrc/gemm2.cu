// Two-SM bf16 GEMM for sm_100a: a cluster of two CTAs computes one 256 x 256 tile of D = A * B^T with
// tcgen05.mma.cta_group::2.  Each CTA stages only its own half of both operands (128 rows of A, 128 rows of B per
// 64-wide k-block: 32 KB per stage instead of the 48 KB a single-CTA 128 x 256 tile needs for the same FLOPs), so
// L2 -> shared-memory traffic per FLOP drops by a third and five pipeline stages fit next to 64 KB of epilogue staging.  The MMA instruction, issued by
// the leader CTA, reads both CTAs' shared memory and writes each CTA's 128 accumulator rows into that CTA's TMEM.
//
// No TMA load uses cluster multicast: each CTA loads its own halves with plain `.cta_group::2` bulk tensor copies
// whose byte counts are credited to the leader's mbarrier.  Stage release and accumulator hand-off use
// tcgen05.commit with `.multicast::cluster` (an mbarrier arrive, not a load).
//
// Supported: forward (A, B K-major; STORE + bias, GELU + pre-activation), dgrad (B MN-major; STORE, DGELU) and wgrad
// (A, B MN-major; bf16 accumulate with deterministic split-K).  Small problems use the single-CTA kernel (gemm.cu).
// Epilogue: sixteen warps per CTA in four groups of four, each group owning 64 columns of the CTA's 128 x 256 half tile
// (64-byte-swizzled staging, TMA stores).
#include "common.cuh"

namespace {

constexpr int BM = 128;               // rows per CTA (256 per pair)
constexpr int BN = 256;               // columns per pair; each CTA stages 128 of them
constexpr int BNH = BN / 2;
constexpr int BK = 64, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_STAGE_BYTES = BNH * BK * 2;           // 16 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_GROUPS = 4;          // epilogue groups of four warps, each owning BN / EPI_GROUPS columns of the tile
constexpr int GROUP_COLS = BN / EPI_GROUPS;
constexpr int EPI_COLS = 32;
constexpr int EPI_BUF_BYTES = BM * EPI_COLS * 2;      // 8 KB
// Staging: 64 KB next to five pipeline stages, split evenly over the sixteen epilogue warps (two 2 KB buffers each).  STORE
// alternates between a warp's two buffers; the epilogues with two tensors per chunk (GELU: activation + pre-activation out;
// dGELU: pre-activation in + gradient out) use one each.
__host__ __device__ constexpr int stages_for(int mode) { return 5; }
__host__ __device__ constexpr int epi_bufs_for(int mode) { return 2 * EPI_GROUPS; }
__host__ __device__ constexpr int smem_for(int mode) { return stages_for(mode) * STAGE_BYTES + epi_bufs_for(mode) * EPI_BUF_BYTES + 1024 + 512; }
constexpr int NUM_THREADS = 576;       // TMA warp + MMA warp + 16 epilogue warps
constexpr int TMEM_COLS = 512;
constexpr int RASTER_GROUP = 8;       // in units of 256-row tiles

enum EpiMode : int { EPI_STORE = 0, EPI_GELU = 1, EPI_DGELU = 2, EPI_ACCUM = 3 };

struct Gemm2Args {
    int M, N, K;
    int num_m_tiles, num_n_tiles, num_kb;     // 256 x 256 tiles
    int splits, kb_per_split;                 // EPI_ACCUM: split-K
    const bf16* bias;
    bf16* D; int ldd;                         // EPI_ACCUM writes D directly
    float* workspace;                         // [half tile][split][128 * 256] fp32 partials
    unsigned int* counters;                   // unused (kept in the argument list of the entry points)
    int accumulate;
    unsigned int* status;
    // optional: flags in this GPU's memory that peers raise when the B operand (gathered weights) is complete
    const unsigned long long* wait_flags; int wait_n; unsigned long long wait_seq; long long wait_cycles;
};

DEVINL bool epi_any(int pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, 512, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(r) : "r"(pred) : "memory");
    return r != 0;
}
DEVINL uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
DEVINL void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
DEVINL uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank)); return r;
}
DEVINL void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-SM bulk tensor load: data lands in this CTA's shared memory, the bytes are credited to the barrier at
// `mbar_cluster_addr` (the leader CTA's).  No multicast.
DEVINL void tma_load_2d_2sm(void* smem_dst, const CUtensorMap* m, uint32_t mbar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(mbar_cluster_addr), "r"(x), "r"(y) : "memory");
}
DEVINL void tmem_alloc_2sm(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
DEVINL void tmem_relinquish_2sm() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
DEVINL void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
DEVINL void umma_ss_2sm(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive (once the MMAs issued so far have completed) on the barrier at this shared-memory offset in both CTAs
DEVINL void umma_commit_2sm(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

template <int A_MN, int B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux, const Gemm2Args g) {
    constexpr int STAGES = stages_for(MODE), NUM_EPI_BUFS = epi_bufs_for(MODE);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + NUM_EPI_BUFS * EPI_BUF_BYTES);
    uint64_t* full = bars;                    // [STAGES]  used in the leader CTA: bytes of both CTAs' loads
    uint64_t* empty = bars + STAGES;          // [STAGES]  one per CTA, raised by the leader's multicast commit
    uint64_t* acc_full = bars + 2 * STAGES;   // [2]       one per CTA, raised by the leader's multicast commit
    uint64_t* acc_empty = acc_full + 2;       // [2]       used in the leader CTA: all epilogue warps of the pair arrive
    uint64_t* aux_full = acc_empty + 2;       // [4 * EPI_GROUPS]  one per epilogue warp (EPI_DGELU)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_full + 4 * EPI_GROUPS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();              // 0 = leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int total_work = g.num_m_tiles * g.num_n_tiles * g.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * 4 * EPI_GROUPS); }
        for (int b = 0; b < 4 * EPI_GROUPS; b++) mbar_init(&aux_full[b], 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
        if (MODE != EPI_ACCUM) tma_prefetch_desc(&tmD);
        if (MODE == EPI_GELU || MODE == EPI_DGELU) tma_prefetch_desc(&tmAux);
    }
    cluster_sync_all();                                   // both CTAs' barriers exist before anyone signals them
    if (warp == 1) { tmem_alloc_2sm(tmem_slot, TMEM_COLS); tmem_relinquish_2sm(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto decode = [&](int w, int& mt, int& nt, int& sp) {
        // split-K: units that run at the same time (consecutive w) cover all tiles of the same K range, so the operand strips of
        // that range are read from DRAM once and shared through the L2; with the split index varying fastest every wave of
        // units streamed whole strips again and the kernel ran at DRAM speed (measured: 0.25 ms against 0.20 for 2304 x 768 x 65536)
        const int tiles = g.num_m_tiles * g.num_n_tiles;
        sp = w / tiles;
        const int t = w - sp * tiles;
        int per_group = RASTER_GROUP * g.num_n_tiles;
        int grp = t / per_group, within = t - grp * per_group;
        int gh = min(RASTER_GROUP, g.num_m_tiles - grp * RASTER_GROUP);
        nt = within / gh;
        mt = grp * RASTER_GROUP + within - nt * gh;
    };

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs; each loads its own halves) ----------------
        if (lane == 0) {
            if (g.wait_flags != nullptr) {
                // The weights this GEMM reads are being gathered from the other GPUs: rank r raises flag r (in this GPU's
                // memory, release at system scope) after its stores have landed.  Bounded polls; on expiry the CTA gives up.
                bool arrived = true;
                for (int r = 0; r < g.wait_n && arrived; r++) {
                    const long long t0 = clock64();
                    while (true) {
                        unsigned long long v;
                        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(g.wait_flags + r) : "memory");
                        if (v >= g.wait_seq) break;
                        if (clock64() - t0 > g.wait_cycles) { record_error(g.status, ST_FLAG_TIMEOUT, 0x9F0 + r); arrived = false; break; }
                        __nanosleep(200);
                    }
                }
                if (!arrived) *abort_flag = 1;
                asm volatile("fence.proxy.async.global;" ::: "memory");      // peers' generic-proxy stores before this thread's TMA loads
            }
            int stage = 0; uint32_t phase = 0;
            for (int w = pair; w < total_work && !*abort_flag; w += npairs) {
                int mt, nt, sp; decode(w, mt, nt, sp);
                const int m0 = mt * 256 + (int)rank * BM;
                const int n0 = nt * BN + (int)rank * BNH;
                const int kb0 = sp * g.kb_per_split, kb1 = min(g.num_kb, kb0 + g.kb_per_split);
                bool fail = false;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, g.status, 0x900 + stage)) { fail = true; break; }
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    uint8_t* sb = sa + A_STAGE_BYTES;
                    const uint32_t lead_full = map_to_cta(smem_u32(&full[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);     // bytes of both CTAs
                    if (A_MN == 0) {
                        tma_load_2d_2sm(sa, &tmA, lead_full, kb * BK, m0);              // box {64 k, 128 rows}
                    } else {
                        #pragma unroll
                        for (int i = 0; i < BM / 64; i++)                                // boxes {64 m, 64 k}
                            tma_load_2d_2sm(sa + i * (BK * 128), &tmA, lead_full, m0 + i * 64, kb * BK);
                    }
                    if (B_MN == 0) {
                        tma_load_2d_2sm(sb, &tmB, lead_full, kb * BK, n0);              // box {64 k, 128 rows}
                    } else {
                        #pragma unroll
                        for (int i = 0; i < BNH / 64; i++)                               // boxes {64 n, 64 k}
                            tma_load_2d_2sm(sb + i * (BK * 128), &tmB, lead_full, n0 + i * 64, kb * BK);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (fail || *abort_flag) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(256, BN, A_MN, B_MN);
            constexpr uint32_t A_STEP = A_MN == 0 ? UMMA_K * 2 : UMMA_K * 128;      // bytes per K step of 16 inside a stage
            constexpr uint32_t B_STEP = B_MN == 0 ? UMMA_K * 2 : UMMA_K * 128;
            const uint64_t da0 = A_MN == 0 ? umma_desc_sw128(smem_u32(smem), 16, 1024) : umma_desc_sw128(smem_u32(smem), BK * 128, 1024);
            const uint64_t db0 = B_MN == 0 ? umma_desc_sw128(smem_u32(smem) + A_STAGE_BYTES, 16, 1024)
                                           : umma_desc_sw128(smem_u32(smem) + A_STAGE_BYTES, BK * 128, 1024);
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            for (int w = pair; w < total_work; w += npairs, it++) {
                int mt, nt, sp; decode(w, mt, nt, sp);
                const int kb0 = sp * g.kb_per_split, kb1 = min(g.num_kb, kb0 + g.kb_per_split);
                const int buf = it & 1;
                const uint32_t use = (uint32_t)(it >> 1);
                if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, g.status, 0xA00 + buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool fail = false;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, g.status, 0xB00 + stage)) { fail = true; break; }
                    tc_fence_after();
                    // descriptors of this stage = those of stage 0 plus the stage offset (the start address sits in the low bits of
                    // a descriptor, in 16-byte units): an instruction costs its issuing thread two additions instead of two
                    // descriptor constructions, which took longer than the product itself runs
                    const uint64_t da_s = da0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
                    const uint64_t db_s = db0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
                    #pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_ss_2sm(d_tmem, da_s + k * (A_STEP >> 4), db_s + k * (B_STEP >> 4), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_2sm(&empty[stage]);      // frees this stage in both CTAs
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (fail) break;
                umma_commit_2sm(&acc_full[buf]);          // both CTAs' accumulator halves are complete
                if (*abort_flag) break;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..17 of each CTA, on that CTA's 128 rows) ----------------
        const int ew = warp - 2;
        const int grp = ew >> 2;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        // Every epilogue warp is its own pipeline over its 32 rows x GROUP_COLS columns: TMEM -> registers -> its own two
        // 2 KB staging buffers (64-byte swizzle) -> its own TMA stores.  Warps never wait for one another, so the TMEM
        // load, shared-memory fence and store-drain latencies of one warp are covered by the other three of its scheduler.
        //   STORE: the two buffers alternate;  GELU: buffer 0 = activation, buffer 1 = pre-activation;
        //   DGELU: buffer 0 = output, buffer 1 = this warp's 32 x 32 box of the stored pre-activation (TMA load).
        constexpr int WARP_BUF_BYTES = 32 * EPI_COLS * 2;           // 2 KB
        static_assert(2 * WARP_BUF_BYTES * 4 * EPI_GROUPS == NUM_EPI_BUFS * EPI_BUF_BYTES, "staging space is split evenly over the epilogue warps");
        uint8_t* wbuf = epi_smem + ew * 2 * WARP_BUF_BYTES;
        constexpr int CHUNKS = GROUP_COLS / EPI_COLS;
        const int swz = (lane >> 1) & 3;
        uint32_t kctr = 0;
        // pre-activation box of chunk c_ of work item w_ -> this warp's second buffer; chunk k completes phase k & 1 of its barrier
        auto aux_load = [&](int w_, int c_) {
            int mt_, nt_, sp_; decode(w_, mt_, nt_, sp_);
            uint64_t* bar = &aux_full[ew];
            mbar_expect_tx(bar, WARP_BUF_BYTES);
            tma_load_2d(wbuf + WARP_BUF_BYTES, &tmAux, bar, nt_ * BN + grp * GROUP_COLS + c_ * EPI_COLS, mt_ * 256 + (int)rank * BM + q * 32);
        };
        // (work item, chunk) that follows (w_, c_) in this warp's sequence; false at the end
        auto next_chunk = [&](int& w_, int& c_) {
            if (c_ + 1 < CHUNKS) { c_++; return true; }
            if (w_ + npairs < total_work) { w_ += npairs; c_ = 0; return true; }
            return false;
        };
        if (MODE == EPI_DGELU && lane == 0 && pair < total_work) aux_load(pair, 0);
        const uint32_t lead_acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
        const uint32_t lead_acc_empty1 = map_to_cta(smem_u32(&acc_empty[1]), 0);
        int it = 0;
        for (int w = pair; w < total_work; w += npairs, it++) {
            int mt, nt, sp; decode(w, mt, nt, sp);
            const int buf = it & 1;
            const uint32_t use = (uint32_t)(it >> 1);
            bool ok = mbar_wait(&acc_full[buf], use & 1, abort_flag, g.status, 0xC00 + buf);
            tc_fence_after();
            const int m0 = mt * 256 + (int)rank * BM, n0 = nt * BN + grp * GROUP_COLS;
            const int grow = m0 + row;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + grp * GROUP_COLS;
            const uint32_t lead_acc_empty = buf ? lead_acc_empty1 : lead_acc_empty0;
            if (MODE == EPI_ACCUM) {
                // ---- EPI_ACCUM: direct global read-modify-write, optional split-K ----
                const int tile = (mt * g.num_n_tiles + nt) * 2 + (int)rank;      // this CTA's half of the 256 x 256 tile
                if (g.splits == 1) {
                    #pragma unroll 1
                    for (int c = 0; c < CHUNKS; c++) {
                        const int col0 = n0 + c * 32;
                        if (col0 >= g.N) break;
                        uint32_t v[32];
                        tmem_ld32(t_row + c * 32, v);
                        tmem_ld_wait();
                        float* f = reinterpret_cast<float*>(v);
                        if (grow < g.M && ok) {
                            #pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                if (col0 + j < g.N) {
                                    bf16* dp = g.D + (size_t)grow * g.ldd + col0 + j;
                                    bf16x8 o;
                                    if (g.accumulate) {
                                        bf16x8 old = ld128(dp);
                                        #pragma unroll
                                        for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(f[j + e] + __bfloat162float(old[e]));
                                    } else {
                                        #pragma unroll
                                        for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(f[j + e]);
                                    }
                                    st128(dp, o);
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
                } else {
                    // partial tile -> workspace, laid out [col/4][row][4] so that a warp writes 512 contiguous bytes
                    float* wsp = g.workspace + ((size_t)tile * g.splits + sp) * (BM * BN);
                    const int cbase = grp * GROUP_COLS;
                    #pragma unroll 1
                    for (int c = 0; c < CHUNKS; c++) {
                        uint32_t v[32];
                        tmem_ld32(t_row + c * 32, v);
                        tmem_ld_wait();
                        #pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j+1]), __uint_as_float(v[j+2]), __uint_as_float(v[j+3]));
                            __stcg(reinterpret_cast<float4*>(wsp + ((size_t)((cbase + c * 32 + j) >> 2) * BM + row) * 4), o);
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
                    // the partial sums of a tile are added, in split order, by gemm2_fold_kernel after this kernel
                }
                if (epi_any(*abort_flag)) break;
                continue;
            }
            #pragma unroll 1
            for (int c = 0; c < CHUNKS; c++) {
                const int col0 = n0 + c * EPI_COLS;
                uint32_t v[32];
                tmem_ld32(t_row + c * EPI_COLS, v);
                tmem_ld_wait();
                if (c == CHUNKS - 1) {
                    // this warp holds the last of its part of the accumulator: tell the leader CTA's MMA thread
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
                }
                float* f = reinterpret_cast<float*>(v);
                if ((MODE == EPI_STORE || MODE == EPI_GELU) && g.bias != nullptr) {
                    #pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col0 + j < g.N) {
                            bf16x8 b = ld128(g.bias + col0 + j);
                            #pragma unroll
                            for (int e = 0; e < 8; e++) f[j + e] += __bfloat162float(b[e]);
                        }
                    }
                }
                uint8_t* out_buf = wbuf + ((MODE == EPI_STORE) ? (kctr & 1) * WARP_BUF_BYTES : 0);
                uint8_t* aux_buf = wbuf + WARP_BUF_BYTES;
                uint8_t* out_row = out_buf + lane * 64;
                uint8_t* aux_row = aux_buf + lane * 64;
                uint4 pre_q[4], out_q[4];
                if (MODE == EPI_DGELU) {
                    ok = mbar_wait(&aux_full[ew], kctr & 1, abort_flag, g.status, 0xC40 + ew) && ok;
                    #pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint4 a = *reinterpret_cast<const uint4*>(aux_row + ((j ^ swz) * 16));
                        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
                        f[j*8+0] *= gelu_grad_fast(a0.x); f[j*8+1] *= gelu_grad_fast(a0.y);
                        f[j*8+2] *= gelu_grad_fast(a1.x); f[j*8+3] *= gelu_grad_fast(a1.y);
                        f[j*8+4] *= gelu_grad_fast(a2.x); f[j*8+5] *= gelu_grad_fast(a2.y);
                        f[j*8+6] *= gelu_grad_fast(a3.x); f[j*8+7] *= gelu_grad_fast(a3.y);
                    }
                    __syncwarp();            // every lane has read its row of the pre-activation box
                    if (lane == 0) {
                        int w_ = w, c_ = c;
                        if (next_chunk(w_, c_)) aux_load(w_, c_);
                    }
                }
                if (MODE == EPI_GELU) {
                    // Two stores per chunk, each from its own buffer and in its own bulk group, issued half a chunk apart:
                    // when a buffer is needed again the only younger group is the other tensor's, so each store has a full
                    // chunk of work to drain underneath (the same slack the alternating buffers give plain STORE).
                    #pragma unroll
                    for (int j = 0; j < 4; j++) {
                        pre_q[j].x = pack_bf16x2(f[j*8+0], f[j*8+1]); pre_q[j].y = pack_bf16x2(f[j*8+2], f[j*8+3]);
                        pre_q[j].z = pack_bf16x2(f[j*8+4], f[j*8+5]); pre_q[j].w = pack_bf16x2(f[j*8+6], f[j*8+7]);
                    }
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    #pragma unroll
                    for (int j = 0; j < 4; j++) *reinterpret_cast<uint4*>(aux_row + ((j ^ swz) * 16)) = pre_q[j];
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0 && ok && col0 < g.N) { tma_store_2d(&tmAux, aux_buf, col0, m0 + q * 32); tma_store_commit(); }
                    #pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // the activation is computed from the rounded pre-activation, so a later recomputation from the stored
                        // tensor gives the same bits
                        const float2 r0 = unpack_bf16x2(pre_q[j].x), r1 = unpack_bf16x2(pre_q[j].y), r2 = unpack_bf16x2(pre_q[j].z), r3 = unpack_bf16x2(pre_q[j].w);
                        out_q[j].x = pack_bf16x2(gelu_fast(r0.x), gelu_fast(r0.y)); out_q[j].y = pack_bf16x2(gelu_fast(r1.x), gelu_fast(r1.y));
                        out_q[j].z = pack_bf16x2(gelu_fast(r2.x), gelu_fast(r2.y)); out_q[j].w = pack_bf16x2(gelu_fast(r3.x), gelu_fast(r3.y));
                    }
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    #pragma unroll
                    for (int j = 0; j < 4; j++) *reinterpret_cast<uint4*>(out_row + ((j ^ swz) * 16)) = out_q[j];
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0 && ok && col0 < g.N) { tma_store_2d(&tmD, out_buf, col0, m0 + q * 32); tma_store_commit(); }
                } else {
                    // all arithmetic happens before the wait for the staging buffer, so the drain of the previous store hides under it
                    #pragma unroll
                    for (int j = 0; j < 4; j++) {
                        out_q[j].x = pack_bf16x2(f[j*8+0], f[j*8+1]); out_q[j].y = pack_bf16x2(f[j*8+2], f[j*8+3]);
                        out_q[j].z = pack_bf16x2(f[j*8+4], f[j*8+5]); out_q[j].w = pack_bf16x2(f[j*8+6], f[j*8+7]);
                    }
                    if (lane == 0) {
                        if (MODE == EPI_STORE) tma_store_wait_read<1>();      // the store issued two chunks ago has read this buffer
                        else tma_store_wait_read<0>();
                    }
                    __syncwarp();
                    #pragma unroll
                    for (int j = 0; j < 4; j++) *reinterpret_cast<uint4*>(out_row + ((j ^ swz) * 16)) = out_q[j];
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0 && ok && col0 < g.N) { tma_store_2d(&tmD, out_buf, col0, m0 + q * 32); tma_store_commit(); }
                }
                kctr++;
            }
            if (epi_any(*abort_flag)) break;
        }
        if (lane == 0) tma_store_wait<0>();
    }

    // teardown: the pair meets (nobody may still signal a barrier of a CTA that has left), then TMEM is freed
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
    }
    cluster_sync_all();
    tc_fence_after();
    if (warp == 1) tmem_dealloc_2sm(tmem_base, TMEM_COLS);
}

// Split-K: D (+)= sum over the splits of the fp32 partial tiles, added in split order (deterministic), one rounding.
// One CTA per 128 x 64 piece of a half tile; a partial is read as it was written ([group of 4 columns][row][4 floats]: a warp
// reads 512 contiguous bytes, every thread has 16 loads of 16 bytes in flight), the sums are transposed through shared
// memory and D is read and written in rows (the 8 lanes of a row move its 128 bytes together).  Folding inside the GEMM by
// the last CTA pair of a tile took 16 dependent round trips to L2 per thread (about 30 us per launch, measured).
__global__ void __launch_bounds__(256)
gemm2_fold_kernel(bf16* __restrict__ D, const float* __restrict__ ws, int M, int N, int ldd, int num_n_tiles, int splits, int accumulate) {
    __shared__ __align__(16) bf16 tile[BM][64 + 8];
    const int chunk = blockIdx.x & 3, half = blockIdx.x >> 2;
    const int rank = half & 1, t2 = half >> 1;
    const int nt = t2 % num_n_tiles, mt = t2 / num_n_tiles;
    const int row0 = mt * 256 + rank * BM, col0 = nt * BN + chunk * 64;
    if (row0 >= M || col0 >= N) return;
    const int t = threadIdx.x;
    const float* src = ws + (size_t)half * splits * (BM * BN) + (size_t)chunk * (16 * BM * 4) + t * 4;
    float4 acc[8];
    #pragma unroll
    for (int k = 0; k < 8; k++) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < splits; sp += 2) {
        const bool two = sp + 1 < splits;
        float4 a0[8], a1[8];
        #pragma unroll
        for (int k = 0; k < 8; k++) a0[k] = __ldcs(reinterpret_cast<const float4*>(src + (size_t)sp * (BM * BN) + k * 1024));
        if (two) {
            #pragma unroll
            for (int k = 0; k < 8; k++) a1[k] = __ldcs(reinterpret_cast<const float4*>(src + (size_t)(sp + 1) * (BM * BN) + k * 1024));
        }
        #pragma unroll
        for (int k = 0; k < 8; k++) { acc[k].x += a0[k].x; acc[k].y += a0[k].y; acc[k].z += a0[k].z; acc[k].w += a0[k].w; }
        if (two) {
            #pragma unroll
            for (int k = 0; k < 8; k++) { acc[k].x += a1[k].x; acc[k].y += a1[k].y; acc[k].z += a1[k].z; acc[k].w += a1[k].w; }
        }
    }
    // thread t holds row t % 128 and the column groups 2k + t / 128 of this piece
    const int row = t & (BM - 1), g0 = t >> 7;
    if (accumulate) {
        // old values first: rows of D into the staging tile, then every thread adds its own elements
        #pragma unroll
        for (int q = 0; q < 4; q++) {
            const int c = q * 256 + t, r = c >> 3, c8 = c & 7;
            uint4 old = make_uint4(0u, 0u, 0u, 0u);
            if (row0 + r < M && col0 + c8 * 8 < N) old = *reinterpret_cast<const uint4*>(D + (size_t)(row0 + r) * ldd + col0 + c8 * 8);
            *reinterpret_cast<uint4*>(&tile[r][c8 * 8]) = old;
        }
        __syncthreads();
    }
    #pragma unroll
    for (int k = 0; k < 8; k++) {
        bf16* p = &tile[row][(2 * k + g0) * 4];
        float o0 = acc[k].x, o1 = acc[k].y, o2 = acc[k].z, o3 = acc[k].w;
        if (accumulate) {
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(p), hi = *reinterpret_cast<const __nv_bfloat162*>(p + 2);
            o0 += __bfloat162float(lo.x); o1 += __bfloat162float(lo.y); o2 += __bfloat162float(hi.x); o3 += __bfloat162float(hi.y);
        }
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(o0, o1);
        *reinterpret_cast<__nv_bfloat162*>(p + 2) = __floats2bfloat162_rn(o2, o3);
    }
    __syncthreads();
    #pragma unroll
    for (int q = 0; q < 4; q++) {
        const int c = q * 256 + t, r = c >> 3, c8 = c & 7;
        if (row0 + r < M && col0 + c8 * 8 < N)
            *reinterpret_cast<uint4*>(D + (size_t)(row0 + r) * ldd + col0 + c8 * 8) = *reinterpret_cast<const uint4*>(&tile[r][c8 * 8]);
    }
}

template <int A_MN, int B_MN, int MODE>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const CUtensorMap& tmAux,
            const Gemm2Args& g, int grid, cudaStream_t stream) {
    static bool configured = false;
    auto kfn = gemm2_kernel<A_MN, B_MN, MODE>;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_for(MODE)));
        configured = true;
    }
    kfn<<<grid, NUM_THREADS, smem_for(MODE), stream>>>(tmA, tmB, tmD, tmAux, g);
    CUDA_CHECK(cudaGetLastError());
    if (MODE == EPI_ACCUM && g.splits > 1) {
        gemm2_fold_kernel<<<g.num_m_tiles * g.num_n_tiles * 2 * 4, 256, 0, stream>>>(g.D, g.workspace, g.M, g.N, g.ldd, g.num_n_tiles, g.splits, g.accumulate);
        CUDA_CHECK(cudaGetLastError());
    }
    return 0;
}

}  // namespace

// Number of fp32 workspace elements and counters llmc_gemm2 needs for a split-K accumulate problem
extern "C" void llmc_gemm2_workspace(int M, int N, int splits, long long* ws_floats, int* num_counters) {
    int halves = CEIL_DIV(M, 256) * CEIL_DIV(N, BN) * 2;
    *ws_floats = splits > 1 ? (long long)halves * splits * BM * BN : 0;
    *num_counters = halves;
}

// Split-K factor for a wgrad-shaped problem.  Model fitted to measurements on 65536-deep products (768..3072 wide): the
// time is waves / s of a whole tile's time plus about 3 % of a tile's time per wave (pipeline fill, partial-tile store and
// the share of the fold kernel); the smallest cost wins, fewer splits on ties.
extern "C" int llmc_gemm2_pick_splits(int M, int N, int K, int sm_count) {
    const int tiles = CEIL_DIV(M, 256) * CEIL_DIV(N, BN), pairs = sm_count / 2, num_kb = CEIL_DIV(K, BK);
    if (tiles >= pairs || num_kb < 16) return 1;
    int best = 1; double best_cost = 1e30;
    for (int s = 1; s <= 16 && s * 8 <= num_kb; s++) {
        const int work = tiles * s, waves = CEIL_DIV(work, pairs);
        const double cost = (double)waves / s + 0.032 * waves;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

// D[M,N] = op(A) * op(B)^T with 256 x 256 tiles on CTA pairs.
//   a_mn_major = 0: A is [M][K]; 1: A is [K][M].   b_mn_major = 0: B is [N][K]; 1: B is [K][N].
// mode: 0 store (+bias), 1 GELU (aux receives the pre-activation), 2 dGELU (aux holds the pre-activation),
//       3 D (+)= result with optional split-K (workspace / counters as sized by llmc_gemm2_workspace).
long long llmc_p2p_wait_cycles_host();      // comm.cu: the limit of every peer-flag wait, in clock cycles

static int gemm2_impl(const bf16* A, const bf16* B, bf16* D, const bf16* bias, bf16* aux, int M, int N, int K,
                      int lda, int ldb, int ldd, int a_mn_major, int b_mn_major, int mode, int accumulate, int splits,
                      float* workspace, unsigned int* counters, const unsigned long long* wait_flags, int wait_n,
                      unsigned long long wait_seq, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldd % 8)) return -1;
    Gemm2Args g;
    g.M = M; g.N = N; g.K = K;
    g.num_m_tiles = CEIL_DIV(M, 256); g.num_n_tiles = CEIL_DIV(N, BN); g.num_kb = CEIL_DIV(K, BK);
    if (mode != EPI_ACCUM || splits < 1) splits = 1;
    if (splits > g.num_kb) splits = g.num_kb;
    g.kb_per_split = CEIL_DIV(g.num_kb, splits);
    g.splits = CEIL_DIV(g.num_kb, g.kb_per_split);
    if (g.splits > 1 && !workspace) return -1;
    g.bias = bias; g.D = D; g.ldd = ldd; g.workspace = workspace; g.counters = counters; g.accumulate = accumulate;
    g.status = llmc_status_ptr();
    g.wait_flags = wait_flags; g.wait_n = wait_n; g.wait_seq = wait_seq; g.wait_cycles = wait_flags ? llmc_p2p_wait_cycles_host() : 0;
    CUtensorMap tmA, tmB, tmD, tmAux;
    int rc;
    if (a_mn_major == 0) {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[2] = {2, (uint64_t)lda * 2};
        uint32_t box[2] = {BK, BM};
        if ((rc = llmc_get_tensormap(&tmA, A, 2, 2, dims, strides, box, 3))) return rc;
    } else {
        uint64_t dims[2] = {(uint64_t)M, (uint64_t)K}, strides[2] = {2, (uint64_t)lda * 2};
        uint32_t box[2] = {64, BK};
        if ((rc = llmc_get_tensormap(&tmA, A, 2, 2, dims, strides, box, 3))) return rc;
    }
    if (b_mn_major == 0) {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)N}, strides[2] = {2, (uint64_t)ldb * 2};
        uint32_t box[2] = {BK, BNH};
        if ((rc = llmc_get_tensormap(&tmB, B, 2, 2, dims, strides, box, 3))) return rc;
    } else {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)K}, strides[2] = {2, (uint64_t)ldb * 2};
        uint32_t box[2] = {64, BK};
        if ((rc = llmc_get_tensormap(&tmB, B, 2, 2, dims, strides, box, 3))) return rc;
    }
    {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[2] = {2, (uint64_t)ldd * 2};
        uint32_t box[2] = {EPI_COLS, 32};        // one epilogue warp's rows
        if ((rc = llmc_get_tensormap(&tmD, D, 2, 2, dims, strides, box, 2))) return rc;
        tmAux = tmD;
        if (mode == EPI_GELU || mode == EPI_DGELU) { if ((rc = llmc_get_tensormap(&tmAux, aux, 2, 2, dims, strides, box, 2))) return rc; }
    }
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    int pairs = sms / 2;
    const int total = g.num_m_tiles * g.num_n_tiles * g.splits;
    if (pairs > total) pairs = total;
    const int grid = 2 * pairs;
#define LAUNCH2(AMJ, BMJ, MD) return launch2<AMJ, BMJ, MD>(tmA, tmB, tmD, tmAux, g, grid, stream)
    if (a_mn_major == 0 && b_mn_major == 0) {
        if (mode == EPI_STORE) LAUNCH2(0, 0, EPI_STORE);
        if (mode == EPI_GELU) LAUNCH2(0, 0, EPI_GELU);
    } else if (a_mn_major == 0 && b_mn_major == 1) {
        if (mode == EPI_STORE) LAUNCH2(0, 1, EPI_STORE);
        if (mode == EPI_DGELU) LAUNCH2(0, 1, EPI_DGELU);
    } else if (a_mn_major == 1 && b_mn_major == 1) {
        if (mode == EPI_ACCUM) LAUNCH2(1, 1, EPI_ACCUM);
    }
#undef LAUNCH2
    return -1;
}

extern "C" int llmc_gemm2(const bf16* A, const bf16* B, bf16* D, const bf16* bias, bf16* aux, int M, int N, int K,
                          int lda, int ldb, int ldd, int a_mn_major, int b_mn_major, int mode, int accumulate, int splits,
                          float* workspace, unsigned int* counters, cudaStream_t stream) {
    return gemm2_impl(A, B, D, bias, aux, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, mode, accumulate, splits, workspace, counters,
                      nullptr, 0, 0, stream);
}

// The same GEMM as the consumer of an in-flight all-gather: before its first load every CTA polls `wait_n` 64-bit flags at
// `wait_flags` (this GPU's memory; rank r's flag is raised by rank r once its shards of the operand have been stored here)
// until they reach `wait_seq`.  The forward pass of early layers then overlaps the update and gather of later ones.
extern "C" int llmc_gemm2_after_flags(const bf16* A, const bf16* B, bf16* D, const bf16* bias, bf16* aux, int M, int N, int K,
                                      int lda, int ldb, int ldd, int a_mn_major, int b_mn_major, int mode, int accumulate, int splits,
                                      float* workspace, unsigned int* counters, const unsigned long long* wait_flags, int wait_n,
                                      unsigned long long wait_seq, cudaStream_t stream) {
    if (wait_flags == nullptr || wait_n < 1 || wait_n > 8) return -1;
    return gemm2_impl(A, B, D, bias, aux, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, mode, accumulate, splits, workspace, counters,
                      wait_flags, wait_n, wait_seq, stream);
}
