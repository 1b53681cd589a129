// bf16 GEMM family for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in TMEM.
//
// One persistent, warp-specialised kernel template covers the three operand layouts a
// transformer needs and their fused epilogues:
//   forward   out = inp * W^T (+ bias) (+ GELU, also emitting the pre-activation)      A K-major,  B K-major
//   dgrad     dinp = dout * W          (* GELU'(pre-activation))                        A K-major,  B MN-major
//   wgrad     dW (+)= dout^T * inp     (split-K, fixed-order reduction, bf16 accumulate) A MN-major, B MN-major
// It replaces the cuBLASLt calls of the reference (llmc/matmul.cuh:109-228 and its epilogues
// BIAS / GELU_AUX_BIAS / DGELU, beta=1 accumulation) with hand-written tcgen05 code.
//
// Structure of a CTA (320 threads, one CTA per SM, tiles taken round-robin):
//   warp 0      TMA producer: fills a 4-stage ring of 128x64 (A) and 256x64 (B) bf16 tiles,
//               128-byte swizzled, signalling `full[stage]` through complete_tx.
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16 four times per stage into one
//               of two 256-column TMEM accumulators and commits to `empty[stage]`; after the last
//               k-block it commits to `acc_full[buf]`.
//   warps 2..9  epilogue, two groups of four warps, each group owning one 128-column half of the tile:
//               tcgen05.ld the accumulator (a warp may touch 32 TMEM lanes = 32 rows), apply the epilogue
//               (the pre-activation of dGELU arrives by TMA), stage bf16 through 64-byte-swizzled shared
//               memory, write with TMA stores, then release the accumulator (`acc_empty[buf]`) so the next
//               tile's MMAs overlap.
// No TMA load uses cluster multicast. All waits are bounded (see common.cuh).
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;            // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_COLS = 32;                          // columns per epilogue chunk (64 B of bf16)
constexpr int EPI_BUF_BYTES = BM * EPI_COLS * 2;      // 8 KB
constexpr int NUM_EPI_BUFS = 4;                       // two per epilogue group
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + NUM_EPI_BUFS * EPI_BUF_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int RASTER_GROUP = 16;
constexpr int MAX_SPLIT_GROUP = 8;

enum EpiMode : int {
    EPI_STORE = 0,      // D = acc (+ bias[n])
    EPI_GELU = 1,       // aux = acc + bias ; D = gelu(aux)
    EPI_DGELU = 2,      // D = acc * gelu'(aux)
    EPI_ACCUM = 3,      // D (+)= acc, optional split-K through a fp32 workspace
};

struct GemmArgs {
    int M, N, K;
    int num_m_tiles, num_n_tiles, splits, kb_per_split, num_kb;
    bf16* D;            // row-major M x N, leading dimension ldd (elements)
    int ldd;
    const bf16* bias;   // N entries or null
    bf16* aux;          // M x N (ldd) pre-activation: written by EPI_GELU, read by EPI_DGELU
    float* workspace;   // split-K partials: [tile][split][BM*BN] fp32
    unsigned int* counters;   // one per tile, zero before the launch, left zero after it
    int accumulate;     // EPI_ACCUM: add to the existing D
    unsigned int* status;
};

DEVINL void epi_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
DEVINL void group_barrier(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory"); }
// barrier over the 256 epilogue threads that also ORs a predicate: every thread gets the same answer
DEVINL bool epi_any(int pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, 256, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(r) : "r"(pred) : "memory");
    return r != 0;
}

template <int A_MN, int B_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + NUM_EPI_BUFS * EPI_BUF_BYTES);
    uint64_t* full = bars;                    // [STAGES]
    uint64_t* empty = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint64_t* aux_full = acc_empty + 2;       // [2] one per epilogue group (EPI_DGELU)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_full + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_work = g.num_m_tiles * g.num_n_tiles * g.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); mbar_init(&aux_full[b], 1); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
        if (MODE != EPI_ACCUM) tma_prefetch_desc(&tmD);
        if (MODE == EPI_GELU || MODE == EPI_DGELU) tma_prefetch_desc(&tmAux);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // work item -> (m tile, n tile, split); m tiles are visited in groups so that concurrently
    // running CTAs share both A and B tiles in L2
    auto decode = [&](int w, int& mt, int& nt, int& sp) {
        sp = w % g.splits;
        int t = w / g.splits;
        int per_group = RASTER_GROUP * g.num_n_tiles;
        int grp = t / per_group, within = t - grp * per_group;
        int gh = min(RASTER_GROUP, g.num_m_tiles - grp * RASTER_GROUP);
        nt = within / gh;
        mt = grp * RASTER_GROUP + within - nt * gh;
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
                int mt, nt, sp; decode(w, mt, nt, sp);
                const int kb0 = sp * g.kb_per_split, kb1 = min(g.num_kb, kb0 + g.kb_per_split);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, g.status, 0x100 + stage)) break;
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    uint8_t* sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(&full[stage], STAGE_BYTES);
                    if (A_MN == 0) {
                        tma_load_2d(sa, &tmA, &full[stage], kb * BK, mt * BM);           // box {64 k, 128 rows}
                    } else {
                        #pragma unroll
                        for (int i = 0; i < BM / 64; i++)                                   // boxes {64 m, 64 k}
                            tma_load_2d(sa + i * (BK * 128), &tmA, &full[stage], mt * BM + i * 64, kb * BK);
                    }
                    if (B_MN == 0) {
                        tma_load_2d(sb, &tmB, &full[stage], kb * BK, nt * BN);           // box {64 k, 256 rows}
                    } else {
                        #pragma unroll
                        for (int i = 0; i < BN / 64; i++)                                   // boxes {64 n, 64 k}
                            tma_load_2d(sb + i * (BK * 128), &tmB, &full[stage], nt * BN + i * 64, kb * BK);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (*abort_flag) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
            constexpr uint32_t A_STEP = A_MN == 0 ? UMMA_K * 2 : UMMA_K * 128;      // bytes per K step of 16 inside a stage
            constexpr uint32_t B_STEP = B_MN == 0 ? UMMA_K * 2 : UMMA_K * 128;
            const uint64_t da0 = A_MN == 0 ? umma_desc_sw128(smem_u32(smem), 16, 1024) : umma_desc_sw128(smem_u32(smem), BK * 128, 1024);
            const uint64_t db0 = B_MN == 0 ? umma_desc_sw128(smem_u32(smem) + A_STAGE_BYTES, 16, 1024)
                                           : umma_desc_sw128(smem_u32(smem) + A_STAGE_BYTES, BK * 128, 1024);
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            for (int w = blockIdx.x; w < total_work; w += gridDim.x, it++) {
                int mt, nt, sp; decode(w, mt, nt, sp);
                const int kb0 = sp * g.kb_per_split, kb1 = min(g.num_kb, kb0 + g.kb_per_split);
                const int buf = it & 1;
                const uint32_t use = (uint32_t)(it >> 1);
                if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, g.status, 0x200 + buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, g.status, 0x300 + stage)) break;
                    tc_fence_after();
                    // descriptors of this stage = those of stage 0 plus the stage offset (the start address sits in the low bits of
                    // a descriptor, in 16-byte units): per instruction the issuing thread does two additions, not two constructions
                    const uint64_t da_s = da0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
                    const uint64_t db_s = db0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
                    #pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_ss(d_tmem, da_s + k * (A_STEP >> 4), db_s + k * (B_STEP >> 4), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[stage]);      // frees the smem stage once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                umma_commit(&acc_full[buf]);          // accumulator complete
                if (*abort_flag) break;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9) ----------------
        // Two groups of four warps; group g owns columns [128 g, 128 g + 128) of the tile and works through them
        // in 32-column chunks staged in 64-byte-swizzled shared memory (two 8 KB buffers per group).
        const int ew = warp - 2;
        const int grp = ew >> 2;
        const int q = warp & 3;                        // TMEM lane quarter this warp may access
        const int row = q * 32 + lane;                 // row of the tile owned by this thread
        const bool leader = ((ew & 3) == 0) && lane == 0;          // issues this group's TMA traffic
        const bool store_thread = (threadIdx.x == 64);             // ACCUM mode: split-K bookkeeping
        uint8_t* bufA = epi_smem + (grp * 2 + 0) * EPI_BUF_BYTES;
        uint8_t* bufB = epi_smem + (grp * 2 + 1) * EPI_BUF_BYTES;
        constexpr int CHUNKS = (BN / 2) / EPI_COLS;
        const int swz = (row >> 1) & 3;                // 64-byte swizzle: 16-byte unit j of row r sits at unit j ^ ((r >> 1) & 3)
        uint8_t* rowA = bufA + row * 64;
        uint8_t* rowB = bufB + row * 64;
        uint32_t kctr = 0;
        auto aux_load = [&](int w_, int c_) {           // pre-activation chunk -> bufB (EPI_DGELU)
            int mt_, nt_, sp_; decode(w_, mt_, nt_, sp_);
            mbar_expect_tx(&aux_full[grp], EPI_BUF_BYTES);
            tma_load_2d(bufB, &tmAux, &aux_full[grp], nt_ * BN + grp * (BN / 2) + c_ * EPI_COLS, mt_ * BM);
        };
        if (MODE == EPI_DGELU && leader && (int)blockIdx.x < total_work) aux_load(blockIdx.x, 0);
        int it = 0;
        for (int w = blockIdx.x; w < total_work; w += gridDim.x, it++) {
            int mt, nt, sp; decode(w, mt, nt, sp);
            const int buf = it & 1;
            const uint32_t use = (uint32_t)(it >> 1);
            bool ok = mbar_wait(&acc_full[buf], use & 1, abort_flag, g.status, 0x400 + buf);
            tc_fence_after();
            const int m0 = mt * BM, n0 = nt * BN + grp * (BN / 2);
            const int grow = m0 + row;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + grp * (BN / 2);

            if (MODE != EPI_ACCUM) {
                #pragma unroll 1
                for (int c = 0; c < CHUNKS; c++) {
                    const int col0 = n0 + c * EPI_COLS;
                    uint32_t v[32];
                    tmem_ld32(t_row + c * EPI_COLS, v);
                    tmem_ld_wait();
                    float* f = reinterpret_cast<float*>(v);
                    if ((MODE == EPI_STORE || MODE == EPI_GELU) && g.bias != nullptr) {
                        #pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (col0 + j < g.N) {   // N is a multiple of 8
                                bf16x8 b = ld128(g.bias + col0 + j);
                                #pragma unroll
                                for (int e = 0; e < 8; e++) f[j + e] += __bfloat162float(b[e]);
                            }
                        }
                    }
                    uint8_t* out_row = rowA;
                    const uint8_t* out_buf = bufA;
                    if (MODE == EPI_STORE) {
                        if (kctr & 1) { out_row = rowB; out_buf = bufB; }
                        if (leader) tma_store_wait_read<1>();      // the store issued two chunks ago has read this buffer
                    } else {
                        if (leader) tma_store_wait_read<0>();
                    }
                    if (MODE == EPI_DGELU) {
                        ok = mbar_wait(&aux_full[grp], kctr & 1, abort_flag, g.status, 0x440 + grp) && ok;
                        #pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint4 a = *reinterpret_cast<const uint4*>(rowB + ((j ^ swz) * 16));
                            const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
                            f[j*8+0] *= gelu_grad_fast(a0.x); f[j*8+1] *= gelu_grad_fast(a0.y);
                            f[j*8+2] *= gelu_grad_fast(a1.x); f[j*8+3] *= gelu_grad_fast(a1.y);
                            f[j*8+4] *= gelu_grad_fast(a2.x); f[j*8+5] *= gelu_grad_fast(a2.y);
                            f[j*8+6] *= gelu_grad_fast(a3.x); f[j*8+7] *= gelu_grad_fast(a3.y);
                        }
                    }
                    group_barrier(grp);      // output buffer is free; (DGELU) everybody has read the pre-activation chunk
                    if (MODE == EPI_DGELU && leader) {
                        if (c + 1 < CHUNKS) aux_load(w, c + 1);
                        else if (w + (int)gridDim.x < total_work) aux_load(w + gridDim.x, 0);
                    }
                    if (MODE == EPI_GELU) {
                        #pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint4 pre, post;
                            pre.x = pack_bf16x2(f[j*8+0], f[j*8+1]); pre.y = pack_bf16x2(f[j*8+2], f[j*8+3]);
                            pre.z = pack_bf16x2(f[j*8+4], f[j*8+5]); pre.w = pack_bf16x2(f[j*8+6], f[j*8+7]);
                            // GELU of the bf16-rounded pre-activation: a later recompute from the stored value gives the same bits
                            const float2 r0 = unpack_bf16x2(pre.x), r1 = unpack_bf16x2(pre.y), r2 = unpack_bf16x2(pre.z), r3 = unpack_bf16x2(pre.w);
                            post.x = pack_bf16x2(gelu_fast(r0.x), gelu_fast(r0.y)); post.y = pack_bf16x2(gelu_fast(r1.x), gelu_fast(r1.y));
                            post.z = pack_bf16x2(gelu_fast(r2.x), gelu_fast(r2.y)); post.w = pack_bf16x2(gelu_fast(r3.x), gelu_fast(r3.y));
                            *reinterpret_cast<uint4*>(rowB + ((j ^ swz) * 16)) = pre;
                            *reinterpret_cast<uint4*>(rowA + ((j ^ swz) * 16)) = post;
                        }
                    } else {
                        #pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint4 o;
                            o.x = pack_bf16x2(f[j*8+0], f[j*8+1]); o.y = pack_bf16x2(f[j*8+2], f[j*8+3]);
                            o.z = pack_bf16x2(f[j*8+4], f[j*8+5]); o.w = pack_bf16x2(f[j*8+6], f[j*8+7]);
                            *reinterpret_cast<uint4*>(out_row + ((j ^ swz) * 16)) = o;
                        }
                    }
                    fence_async_smem();
                    group_barrier(grp);
                    if (leader && ok && col0 < g.N) {
                        tma_store_2d(&tmD, out_buf, col0, m0);
                        if (MODE == EPI_GELU) tma_store_2d(&tmAux, bufB, col0, m0);
                        tma_store_commit();
                    }
                    kctr++;
                }
                // accumulator fully read: hand it back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            } else {
                // ---- EPI_ACCUM: direct global read-modify-write, optional split-K ----
                const int tile = mt * g.num_n_tiles + nt;
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
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                } else {
                    // partial tile -> workspace, laid out [col/4][row][4] so that a warp writes 512 contiguous bytes
                    float* wsp = g.workspace + ((size_t)tile * g.splits + sp) * (BM * BN);
                    const int cbase = grp * (BN / 2);
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
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                    __threadfence();
                    epi_barrier();
                    if (store_thread) {
                        unsigned int prev = atomicAdd(&g.counters[tile], 1u);
                        *last_flag = (prev == (unsigned int)(g.splits - 1));
                        if (prev == (unsigned int)(g.splits - 1)) g.counters[tile] = 0;   // ready for the next launch
                    }
                    epi_barrier();
                    if (*last_flag && ok) {
                        __threadfence();
                        const float* wt = g.workspace + (size_t)tile * g.splits * (BM * BN);
                        if (grow < g.M) {
                            #pragma unroll 1
                            for (int jj = 0; jj < BN / 2; jj += 8) {
                                const int j = cbase + jj;              // column inside the tile
                                if (nt * BN + j >= g.N) break;
                                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                                // all loads of a group of splits are issued before the adds (memory-level parallelism);
                                // the adds run in split order: deterministic
                                for (int s0 = 0; s0 < g.splits; s0 += MAX_SPLIT_GROUP) {
                                    float4 va[MAX_SPLIT_GROUP], vb[MAX_SPLIT_GROUP];
                                    #pragma unroll
                                    for (int s = 0; s < MAX_SPLIT_GROUP; s++) {
                                        if (s0 + s < g.splits) {
                                            const float* p = wt + (size_t)(s0 + s) * (BM * BN);
                                            va[s] = __ldcg(reinterpret_cast<const float4*>(p + ((size_t)(j >> 2) * BM + row) * 4));
                                            vb[s] = __ldcg(reinterpret_cast<const float4*>(p + ((size_t)((j >> 2) + 1) * BM + row) * 4));
                                        }
                                    }
                                    #pragma unroll
                                    for (int s = 0; s < MAX_SPLIT_GROUP; s++) {
                                        if (s0 + s < g.splits) {
                                            acc[0] += va[s].x; acc[1] += va[s].y; acc[2] += va[s].z; acc[3] += va[s].w;
                                            acc[4] += vb[s].x; acc[5] += vb[s].y; acc[6] += vb[s].z; acc[7] += vb[s].w;
                                        }
                                    }
                                }
                                bf16* dp = g.D + (size_t)grow * g.ldd + nt * BN + j;
                                bf16x8 o;
                                if (g.accumulate) {
                                    bf16x8 old = ld128(dp);
                                    #pragma unroll
                                    for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(acc[e] + __bfloat162float(old[e]));
                                } else {
                                    #pragma unroll
                                    for (int e = 0; e < 8; e++) o[e] = __float2bfloat16_rn(acc[e]);
                                }
                                st128(dp, o);
                            }
                        }
                    }
                    epi_barrier();   // last_flag is rewritten by the next tile
                }
            }
            if (epi_any(*abort_flag)) break;   // uniform decision: nobody is left alone at a barrier
        }
        if (leader) tma_store_wait<0>();
    }

    // teardown: everybody meets, then the allocating warp frees TMEM
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {
        // a wait was abandoned: give copies that are still in flight time to land before the CTA's
        // shared memory is released
        long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

int make_operand_map(CUtensorMap* tm, const bf16* ptr, int mn_major, int mn_extent, int k_extent, int ld, int tile_mn) {
    uint64_t dims[2], strides[2]; uint32_t box[2];
    if (mn_major == 0) {            // stored [mn][k], k contiguous
        dims[0] = (uint64_t)k_extent; dims[1] = (uint64_t)mn_extent;
        box[0] = BK; box[1] = (uint32_t)tile_mn;
    } else {                        // stored [k][mn], mn contiguous
        dims[0] = (uint64_t)mn_extent; dims[1] = (uint64_t)k_extent;
        box[0] = 64; box[1] = BK;
    }
    strides[0] = 2; strides[1] = (uint64_t)ld * 2;
    return llmc_get_tensormap(tm, ptr, 2, 2, dims, strides, box, 3);
}

template <int A_MN, int B_MN, int MODE>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const CUtensorMap& tmAux,
           const GemmArgs& g, int grid, cudaStream_t stream) {
    static bool configured = false;
    auto kfn = gemm_kernel<A_MN, B_MN, MODE>;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    kfn<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmD, tmAux, g);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

}  // namespace

// Number of fp32 workspace elements and counters llmc_gemm needs for a given problem
extern "C" void llmc_gemm_workspace(int M, int N, int splits, long long* ws_floats, int* num_counters) {
    int tiles = CEIL_DIV(M, BM) * CEIL_DIV(N, BN);
    *ws_floats = splits > 1 ? (long long)tiles * splits * BM * BN : 0;
    *num_counters = tiles;
}

// Pick a split-K factor that fills the machine for a wgrad-shaped problem
extern "C" int llmc_gemm_pick_splits(int M, int N, int K, int sm_count) {
    int tiles = CEIL_DIV(M, BM) * CEIL_DIV(N, BN);
    int num_kb = CEIL_DIV(K, BK);
    if (tiles >= sm_count || num_kb < 16) return 1;
    int best = 1; double best_eff = 0.0;
    for (int s = 1; s <= 8 && s * 8 <= num_kb; s++) {
        int work = tiles * s;
        int waves = CEIL_DIV(work, sm_count);
        double eff = (double)work / ((double)waves * sm_count);
        // splitting costs a workspace round trip: prefer fewer splits on ties
        if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    }
    return best;
}

// D[M,N] = op(A) * op(B)^T with the epilogue selected by `mode` (EpiMode).
//   a_mn_major = 0: A is stored [M][K] (lda = row stride);  1: stored [K][M]
//   b_mn_major = 0: B is stored [N][K] (ldb = row stride);  1: stored [K][N]
// All leading dimensions in elements and multiples of 8; pointers 16-byte aligned.
extern "C" int llmc_gemm(const bf16* A, const bf16* B, bf16* D, const bf16* bias, bf16* aux,
                         int M, int N, int K, int lda, int ldb, int ldd,
                         int a_mn_major, int b_mn_major, int mode, int accumulate,
                         int splits, float* workspace, unsigned int* counters,
                         int max_ctas, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldd % 8)) { fprintf(stderr, "[llmc_b200] gemm: N and leading dimensions must be multiples of 8\n"); return -1; }
    GemmArgs g;
    g.M = M; g.N = N; g.K = K;
    g.num_m_tiles = CEIL_DIV(M, BM); g.num_n_tiles = CEIL_DIV(N, BN);
    g.num_kb = CEIL_DIV(K, BK);
    if (mode != EPI_ACCUM || splits < 1) splits = 1;
    if (splits > g.num_kb) splits = g.num_kb;
    g.kb_per_split = CEIL_DIV(g.num_kb, splits);
    splits = CEIL_DIV(g.num_kb, g.kb_per_split);      // no empty split
    g.splits = splits;
    if (splits > 1 && (workspace == nullptr || counters == nullptr)) { fprintf(stderr, "[llmc_b200] gemm: split-K needs workspace\n"); return -1; }
    g.D = D; g.ldd = ldd; g.bias = bias; g.aux = aux; g.workspace = workspace; g.counters = counters;
    g.accumulate = accumulate;
    g.status = llmc_status_ptr();

    CUtensorMap tmA, tmB, tmD, tmAux;
    int rc;
    if ((rc = make_operand_map(&tmA, A, a_mn_major, M, K, lda, BM))) return rc;
    if ((rc = make_operand_map(&tmB, B, b_mn_major, N, K, ldb, BN))) return rc;
    {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[2] = {2, (uint64_t)ldd * 2};
        uint32_t box[2] = {EPI_COLS, BM};
        if ((rc = llmc_get_tensormap(&tmD, D, 2, 2, dims, strides, box, 2))) return rc;       // 64-byte swizzle
        tmAux = tmD;
        if (mode == EPI_GELU || mode == EPI_DGELU) { if ((rc = llmc_get_tensormap(&tmAux, aux, 2, 2, dims, strides, box, 2))) return rc; }
    }
    int sms = llmc_device_sm_count();
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    int total = g.num_m_tiles * g.num_n_tiles * g.splits;
    int grid = total < sms ? total : sms;
    if (grid < 1) grid = 1;

#define LAUNCH(AM, BMj, MD) return launch<AM, BMj, MD>(tmA, tmB, tmD, tmAux, g, grid, stream)
    if (a_mn_major == 0 && b_mn_major == 0) {
        if (mode == EPI_STORE) LAUNCH(0, 0, EPI_STORE);
        if (mode == EPI_GELU) LAUNCH(0, 0, EPI_GELU);
        if (mode == EPI_ACCUM) LAUNCH(0, 0, EPI_ACCUM);
    } else if (a_mn_major == 0 && b_mn_major == 1) {
        if (mode == EPI_STORE) LAUNCH(0, 1, EPI_STORE);
        if (mode == EPI_DGELU) LAUNCH(0, 1, EPI_DGELU);
    } else if (a_mn_major == 1 && b_mn_major == 1) {
        if (mode == EPI_ACCUM) LAUNCH(1, 1, EPI_ACCUM);
        if (mode == EPI_STORE) LAUNCH(1, 1, EPI_STORE);
    }
#undef LAUNCH
    fprintf(stderr, "[llmc_b200] gemm: unsupported layout/mode combination (%d,%d,%d)\n", a_mn_major, b_mn_major, mode);
    return -1;
}
