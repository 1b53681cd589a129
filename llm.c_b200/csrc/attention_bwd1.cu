// Causal flash attention backward for sm_100a, head size 64, on the packed (B, T, 3, NH, HS) layout: ONE pass over the
// (key tile j, query tile i) pairs with the five products of the algorithm and nothing recomputed.
//
// The score tiles are formed TRANSPOSED (key rows on the TMEM lanes, queries along the columns), so that the two products
// that accumulate over the query loop take their A operand straight from tensor memory:
//
//   S^T  = K_j Q_i^T          dP^T = V_j dO_i^T                    (SS products, 128 x 128 fp32 in TMEM)
//   P^T  = exp(S^T scale - LSE_q)     dS^T = P^T (dP^T - delta_q) scale      (softmax threads; bf16 back into TMEM,
//                                                                             dS^T also to shared memory)
//   dV_j += P^T dO_i          dK_j += dS^T Q_i                     (TS products: A from TMEM, B = the streamed tile)
//   dQ_i(j) = dS K_j                                               (SS product: A = dS^T read M-major from shared memory)
//
// Shared-memory bandwidth is what bounds such a kernel at 64-wide heads (a 128 x 64 x 16 product with both operands in
// shared memory reads 6 KB for 32 cycles of arithmetic); keeping P^T and dS^T in tensor memory removes a third of that
// traffic and all of the P stores.
//
// A work item is (batch, head, g) with the two key tiles {g, nt-1-g}: nt + 1 pairs whatever g, so a static round-robin over
// the persistent CTAs is balanced.  dK_j / dV_j leave the CTA once per key tile.  The contribution of pair (j, i) to dQ_i is
// written as fp32 to its own slot of a workspace; a second kernel adds the slots of a query tile in the order j = 0..i and
// rounds once.  No atomics, no ordering between CTAs: the gradients are bit-reproducible, which the reference also demands of
// cuDNN (llmc/cudnn_att.cpp:186-191), and no CTA ever waits for another one.
//
// Roles inside a CTA (512 threads):
//   warp 0       TMA producer: K_j, V_j resident (double buffered across key tiles); Q_i, dO_i through a 3-stage ring.
//   warp 1       issuer of all five products, in the order dV(t), S^T(t+1), dK(t), dQ(t), dP^T(t+1): program order is what
//                keeps dP^T of the next pair from overwriting the bf16 dS^T operand that aliases its TMEM columns.
//   warps 4-11   softmax: thread = key row x 64-query half.  Nothing is exchanged between threads (the row statistics of the
//                forward pass are per query = per column, read from a small shared table).
//   warps 12-15  drain: the pair's dQ contribution from TMEM to the workspace, and at the end of a key tile dV_j / dK_j to
//                global memory through a staging buffer and TMA stores; also producers of the per-query statistics table.
//
// TMEM columns: S^T [0,128)  dP^T [128,256) (dS^T bf16 aliases the first 32 columns of each 64-column half)
//               dV [256,320)  dK [320,384)  dQ [384,448)  P^T bf16 [448,512).
//
// Head sizes above 64 use the two-pass kernels of attention_bwd.cu.
//
// Capability parity: attention_backward_cudnn (llmc/cudnn_att.cpp:256-288) and attention_backward of llmc/attention.cuh.
#include "common.cuh"

int llmc_attn_qkv_map(CUtensorMap* tm, const bf16* qkv, int B, int T, int NH, int hs);   // attention_fwd.cu
int llmc_attention_bwd_two_pass(bf16* dqkv, float* delta, const bf16* dout, const bf16* qkv, const bf16* out, const float* lse,
                                int B, int T, int NH, int hs, cudaStream_t stream);      // attention_bwd.cu
int llmc_attention_delta(float* delta, const bf16* out, const bf16* dout, int B, int T, int NH, int hs, cudaStream_t stream);

namespace {

constexpr int BT = 128;                             // tile rows (queries and keys)
constexpr int HS = 64;
constexpr int TILE_BYTES = BT * HS * 2;             // 16 KB: one 128-byte-swizzled TMA box
constexpr int PAIR_BYTES = 2 * TILE_BYTES;
constexpr int DS_BYTES = BT * BT * 2;               // 32 KB
constexpr int RB = 2;                               // resident (K_j, V_j) buffers
constexpr int XSTAGES = 3;                          // ring of streamed (Q_i, dO_i) pairs
constexpr int THREADS = 512;
constexpr int TMEM_COLS = 512;
constexpr int STAT_BYTES = 2 * 2 * BT * 4;          // [2 buffers][lse, delta][128 queries]
constexpr int SMEM = RB * PAIR_BYTES + XSTAGES * PAIR_BYTES + DS_BYTES + PAIR_BYTES + STAT_BYTES + 256;
constexpr int SLOT_FLOATS = BT * HS;                // one dQ contribution
static_assert(SMEM <= 232448, "shared memory of one CTA");

struct Args {
    bf16* dqkv;          // (B, T, 3, NH, 64)
    float* dq_ws;        // [B*NH][nt*(nt+1)/2][16 column groups][128 rows][4] fp32: slot of pair (j, i) = i*(i+1)/2 + j
    const float* lse;    // (B, NH, T)
    const float* delta;  // (B, NH, T)
    int B, T, NH;
    float scale, scale_log2e;
    unsigned int* status;
    long long* trace;    // optional: [4 roles][8 events][TRACE_PAIRS] clock64() stamps of CTA 0 (null in normal runs)
};
constexpr int TRACE_PAIRS = 64;

DEVINL void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
DEVINL void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

// The sequence of pairs of one CTA: items w (round-robin), their one or two key tiles, the query tiles i >= j of each.
struct Walk {
    int w, total, G, nt, stride, NH;
    int bh, b, h, g, seg, j, i;
    DEVINL void start(int first, int total_, int G_, int nt_, int stride_, int NH_) {
        w = first; total = total_; G = G_; nt = nt_; stride = stride_; NH = NH_;
        bh = b = h = g = seg = j = i = 0;
        if (w < total) item();
    }
    DEVINL bool valid() const { return w < total; }
    DEVINL void item() { bh = w / G; g = w - bh * G; b = bh / NH; h = bh - b * NH; seg = 0; j = g; i = j; }
    DEVINL bool first_of_tile() const { return i == j; }
    DEVINL bool last_of_tile() const { return i == nt - 1; }
    DEVINL void next() {                      // valid() turns false past the last pair
        if (++i < nt) return;
        if (seg == 0 && 2 * g != nt - 1) { seg = 1; j = nt - 1 - g; i = j; return; }
        w += stride;
        if (w < total) item();
    }
};

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd1_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQKV, const Args a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sRes = smem;                              // [RB][K_j, V_j]
    uint8_t* sStr = sRes + RB * PAIR_BYTES;            // [XSTAGES][Q_i, dO_i]
    uint8_t* sdS = sStr + XSTAGES * PAIR_BYTES;        // dS^T: 128 key rows x 128 queries, two 64-query chunks of 128-byte rows
    uint8_t* sOut = sdS + DS_BYTES;                    // dV_j, dK_j on their way out (two TMA boxes)
    float* sStat = reinterpret_cast<float*>(sOut + PAIR_BYTES);     // [2][2][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStat) + STAT_BYTES);
    uint64_t* res_full = bars + 0;    // [2]
    uint64_t* res_empty = bars + 2;   // [2]
    uint64_t* x_full = bars + 4;      // [3]
    uint64_t* x_empty = bars + 7;     // [3]
    uint64_t* s_full = bars + 10;     // S^T(t) complete                            (1 commit)
    uint64_t* s_empty = bars + 11;    // every softmax warp has S^T(t) in registers  (8 arrivals)
    uint64_t* dp_full = bars + 12;    // dP^T(t) complete                           (1 commit)
    uint64_t* p_ready = bars + 13;    // P^T(t) is in TMEM                           (8 arrivals)
    uint64_t* p_empty = bars + 14;    // dV(t) has read P^T(t)                       (1 commit)
    uint64_t* ds_ready = bars + 15;   // dS^T(t) is in TMEM and in shared memory     (8 arrivals)
    uint64_t* ds_empty = bars + 16;   // dK(t), dQ(t) have read dS^T(t)              (1 commit)
    uint64_t* dq_full = bars + 17;    // dQ(t) complete                              (1 commit)
    uint64_t* dq_empty = bars + 18;   // the drain warps hold dQ(t) in registers     (4 arrivals)
    uint64_t* acc_full = bars + 19;   // dV_j, dK_j complete                         (1 commit)
    uint64_t* acc_empty = bars + 20;  // the drain warps hold them                   (4 arrivals)
    uint64_t* st_full = bars + 21;    // [2] statistics table of a pair written      (4 arrivals)
    uint64_t* st_empty = bars + 23;   // [2] ... and read by every softmax warp      (8 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = CEIL_DIV(a.T, BT);
    const int G = (nt + 1) >> 1;                      // key-tile groups {g, nt-1-g}
    const int total = a.B * a.NH * G;
    const int npairs = nt * (nt + 1) / 2;

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) record_error(a.status, ST_BAD_ARG, 0x28);
        for (int i = 0; i < 2; i++) { mbar_init(&res_full[i], 1); mbar_init(&res_empty[i], 1); mbar_init(&st_full[i], 4); mbar_init(&st_empty[i], 8); }
        for (int i = 0; i < XSTAGES; i++) { mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1); }
        mbar_init(s_full, 1); mbar_init(s_empty, 8); mbar_init(dp_full, 1); mbar_init(p_ready, 8); mbar_init(p_empty, 1);
        mbar_init(ds_ready, 8); mbar_init(ds_empty, 1); mbar_init(dq_full, 1); mbar_init(dq_empty, 4);
        mbar_init(acc_full, 1); mbar_init(acc_empty, 4);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmDQKV);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 320, tdQ = tmem_base + 384,
                   tP = tmem_base + 448;

    // time stamps of CTA 0's first TRACE_PAIRS pairs, one thread per role, for the timeline tool (llmc_attention_bwd_set_trace)
#define TRACE(role, ev) do { if (a.trace != nullptr && blockIdx.x == 0 && t < TRACE_PAIRS) a.trace[((role) * 8 + (ev)) * TRACE_PAIRS + t] = clock64(); } while (0)

    Walk wk;
    wk.start(blockIdx.x, total, G, nt, gridDim.x, a.NH);

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int xst = 0; uint32_t xph = 0;
            int kvt = 0;
            for (; wk.valid(); wk.next()) {
                if (wk.first_of_tile()) {
                    const int rb = kvt & 1;
                    if (!mbar_wait_relaxed(&res_empty[rb], ((kvt >> 1) & 1) ^ 1, abort_flag, a.status, 0x681)) break;
                    uint8_t* rdst = sRes + rb * PAIR_BYTES;
                    mbar_expect_tx(&res_full[rb], PAIR_BYTES);
                    tma_load_4d(rdst, &tmQKV, &res_full[rb], 0, a.NH + wk.h, wk.j * BT, wk.b);                    // K_j
                    tma_load_4d(rdst + TILE_BYTES, &tmQKV, &res_full[rb], 0, 2 * a.NH + wk.h, wk.j * BT, wk.b);   // V_j
                    kvt++;
                }
                if (!mbar_wait_relaxed(&x_empty[xst], xph ^ 1, abort_flag, a.status, 0x680)) break;
                uint8_t* dst = sStr + xst * PAIR_BYTES;
                mbar_expect_tx(&x_full[xst], PAIR_BYTES);
                tma_load_4d(dst, &tmQKV, &x_full[xst], 0, wk.h, wk.i * BT, wk.b);                                 // Q_i
                tma_load_4d(dst + TILE_BYTES, &tmDO, &x_full[xst], 0, wk.h, wk.i * BT, wk.b);                     // dO_i
                if (++xst == XSTAGES) { xst = 0; xph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- issuer of the five products
        // The whole warp runs this code in uniform control flow and one elected lane executes the tcgen05 instructions.  With a
        // single lane inside a divergent branch every descriptor has to be moved from that lane's registers to uniform registers,
        // which costs the issuing thread about 90 cycles per product (measured) -- more than a 128 x 64 x 16 product runs.
        // Wait results go through a warp vote so that the compiler knows the branches on them to be uniform.
        if (wk.valid()) {
            const bool leader = elect_one();
#define WAIT_ALL(bar, parity, code) (__all_sync(0xffffffffu, mbar_wait_relaxed(bar, parity, abort_flag, a.status, code, 32)) != 0)
            constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BT, 0, 0);      // S^T, dP^T: both operands K-major
            constexpr uint32_t idesc_ts = umma_idesc_bf16(BT, HS, 0, 1);     // dV, dK: A from TMEM, B N-major
            constexpr uint32_t idesc_q = umma_idesc_bf16(BT, HS, 1, 1);      // dQ: A = dS^T read M-major, B = K_j N-major
            // Descriptors of buffer 0 of each kind are built once; the others follow by addition (the start address sits in the
            // low bits of a descriptor, in 16-byte units).
            const uint64_t dQk0 = umma_desc_sw128(smem_u32(sStr), 16, 1024), dOk0 = umma_desc_sw128(smem_u32(sStr + TILE_BYTES), 16, 1024);
            const uint64_t dQn0 = umma_desc_sw128(smem_u32(sStr), TILE_BYTES, 1024), dOn0 = umma_desc_sw128(smem_u32(sStr + TILE_BYTES), TILE_BYTES, 1024);
            const uint64_t dKk0 = umma_desc_sw128(smem_u32(sRes), 16, 1024), dVk0 = umma_desc_sw128(smem_u32(sRes + TILE_BYTES), 16, 1024);
            const uint64_t dKn0 = umma_desc_sw128(smem_u32(sRes), TILE_BYTES, 1024);
            const uint64_t dSm = umma_desc_sw128(smem_u32(sdS), BT * 128, 1024);     // dS^T as an M-major A operand
            constexpr uint32_t PAIR_UNITS = PAIR_BYTES / 16;
            // S^T and dP^T of one pair: A = resident K_j / V_j, B = streamed Q_i / dO_i; 16 channels = 32 bytes = 2 address units per step
            auto issue_s = [&](int rb, int st) {
                const uint64_t ka = dKk0 + (uint32_t)rb * PAIR_UNITS, qb = dQk0 + (uint32_t)st * PAIR_UNITS;
                if (leader) {
                    #pragma unroll
                    for (int kk = 0; kk < HS / 16; kk++) umma_ss(tS, ka + 2 * kk, qb + 2 * kk, idesc_s, kk > 0);
                    umma_commit(s_full);
                }
            };
            auto issue_dp = [&](int rb, int st) {
                const uint64_t va = dVk0 + (uint32_t)rb * PAIR_UNITS, ob = dOk0 + (uint32_t)st * PAIR_UNITS;
                if (leader) {
                    #pragma unroll
                    for (int kk = 0; kk < HS / 16; kk++) umma_ss(tdP, va + 2 * kk, ob + 2 * kk, idesc_s, kk > 0);
                    umma_commit(dp_full);
                }
            };
            uint32_t t = 0;
            int st = 0;                // ring stage of pair t
            uint32_t xph = 0;          // parity of the ring round of pair t
            int kvt = 0;               // key-tile counter of pair t
            // prologue: S^T(0), dP^T(0)
            bool ok = WAIT_ALL(&res_full[0], 0, 0x690) && WAIT_ALL(&x_full[0], 0, 0x691);
            tc_fence_after();
            if (ok) { issue_s(0, 0); issue_dp(0, 0); }
            while (ok) {
                // pair t = wk; the pair after it, if any
                Walk nx = wk; nx.next();
                const bool have_next = nx.valid();
                const int rb = kvt & 1;
                const int nst = st + 1 == XSTAGES ? 0 : st + 1;
                const uint32_t nph = st + 1 == XSTAGES ? xph ^ 1 : xph;
                const int nkvt = have_next && nx.first_of_tile() ? kvt + 1 : kvt;
                const int nrb = nkvt & 1;
                const uint32_t acc = wk.first_of_tile() ? 0u : 1u;
                // ---- dV(t) += P^T dO_i : A = P^T in TMEM (16 queries = 8 columns per step), B = dO_i N-major (16 rows = 2048 bytes)
                if (leader) TRACE(0, 0);
                ok = WAIT_ALL(p_ready, t & 1, 0x692);
                if (ok && wk.first_of_tile() && kvt > 0) ok = WAIT_ALL(acc_empty, (kvt - 1) & 1, 0x693);
                if (!ok) break;
                tc_fence_after();
                if (leader) TRACE(0, 1);
                {
                    const uint64_t ob = dOn0 + (uint32_t)st * PAIR_UNITS;
                    if (leader) {
                        #pragma unroll
                        for (int kk = 0; kk < BT / 16; kk++) umma_ts(tdV, tP + kk * 8, ob + 128 * kk, idesc_ts, acc | (kk > 0));
                        umma_commit(p_empty);
                    }
                }
                // ---- S^T(t+1): its TMEM tile was read into registers before P^T(t) could be written
                if (have_next) {
                    if (nx.first_of_tile()) ok = WAIT_ALL(&res_full[nrb], (nkvt >> 1) & 1, 0x694);
                    ok = ok && WAIT_ALL(&x_full[nst], nph, 0x695);
                    ok = ok && WAIT_ALL(s_empty, t & 1, 0x696);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(nrb, nst);
                }
                if (leader) TRACE(0, 2);
                // ---- dK(t) += dS^T Q_i (A = dS^T in TMEM: queries 0..63 in columns [0,32) of the dP^T tile, 64..127 in [64,96));
                //      dQ(t) = dS K_j (A = dS^T in shared memory read M-major: 16 key rows = 2048 bytes per step)
                ok = WAIT_ALL(ds_ready, t & 1, 0x697);
                if (ok && t > 0) ok = WAIT_ALL(dq_empty, (t - 1) & 1, 0x698);
                if (!ok) break;
                tc_fence_after();
                if (leader) TRACE(0, 3);
                {
                    const uint64_t qb = dQn0 + (uint32_t)st * PAIR_UNITS, kb = dKn0 + (uint32_t)rb * PAIR_UNITS;
                    if (leader) {
                        #pragma unroll
                        for (int kk = 0; kk < BT / 16; kk++)
                            umma_ts(tdK, tdP + (kk >> 2) * 64 + (kk & 3) * 8, qb + 128 * kk, idesc_ts, acc | (kk > 0));
                        #pragma unroll
                        for (int kk = 0; kk < BT / 16; kk++) umma_ss(tdQ, dSm + 128 * kk, kb + 128 * kk, idesc_q, kk > 0);
                        umma_commit(dq_full);
                        umma_commit(ds_empty);
                        umma_commit(&x_empty[st]);
                        if (wk.last_of_tile()) { umma_commit(acc_full); umma_commit(&res_empty[rb]); }
                    }
                }
                // ---- dP^T(t+1): after dK(t) in program order, so it cannot overwrite dS^T(t) early
                if (have_next) issue_dp(nrb, nst);
                if (leader) TRACE(0, 4);
                if (!have_next) break;
                wk = nx; st = nst; xph = nph; kvt = nkvt; t++;
            }
#undef WAIT_ALL
        }
    } else if (warp >= 4 && warp < 12) {
        // ---------------------------------------------------------------- softmax: thread = key row r x query half hf
        const int q = warp & 3;                        // TMEM lane quarter
        const int hf = (warp - 4) >> 2;                // query half
        const int r = q * 32 + lane;                   // key row of the tile
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        bool ok = true;
        uint32_t t = 0;
        for (; wk.valid(); wk.next(), t++) {
            const int i = wk.i, j = wk.j;
            const bool row_ok = j * BT + r < a.T;
            const float* stat = sStat + (t & 1) * (2 * BT) + hf * 64;       // lse * log2(e) of this half's queries; delta * scale 128 floats further
            if (threadIdx.x == 128) TRACE(1, 0);
            ok = mbar_wait(s_full, t & 1, abort_flag, a.status, 0x6a0) && ok;
            tc_fence_after();
            if (threadIdx.x == 128) TRACE(1, 1);
            ok = mbar_wait(&st_full[t & 1], (t >> 1) & 1, abort_flag, a.status, 0x6a1) && ok;
            if (t > 0) ok = mbar_wait(p_empty, (t - 1) & 1, abort_flag, a.status, 0x6a2) && ok;      // dV(t-1) has read P^T(t-1)
            if (threadIdx.x == 128) TRACE(1, 7);
            // ---- P^T = exp2(S^T * scale * log2(e) - LSE * log2(e)); causal: query >= key.  Two passes of 32 queries: with all 64
            //      scores in registers next to the 64 results the register file is so full that the compiler reuses registers
            //      across the exponentials, and every one then waits for its predecessor (measured: 34 cycles per element).
            float p[64];
            // only the diagonal tile and a ragged last key tile need masks; both conditions are the same for the whole warp
            const bool masked = (i == j) || (j * BT + BT > a.T);
            #pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                uint32_t sv[32];
                tmem_ld32(tS + lane_off + hf * 64 + h2 * 32, sv);
                tmem_ld_wait();
                if (h2 == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s_empty);
                    if (threadIdx.x == 128) TRACE(1, 6);
                }
                if (!masked) {
                    #pragma unroll
                    for (int e4 = 0; e4 < 8; e4++) {
                        const float4 l4 = *reinterpret_cast<const float4*>(stat + h2 * 32 + e4 * 4);
                        p[h2 * 32 + e4 * 4 + 0] = ex2_fast(fmaf(__uint_as_float(sv[e4 * 4 + 0]), a.scale_log2e, -l4.x));
                        p[h2 * 32 + e4 * 4 + 1] = ex2_fast(fmaf(__uint_as_float(sv[e4 * 4 + 1]), a.scale_log2e, -l4.y));
                        p[h2 * 32 + e4 * 4 + 2] = ex2_fast(fmaf(__uint_as_float(sv[e4 * 4 + 2]), a.scale_log2e, -l4.z));
                        p[h2 * 32 + e4 * 4 + 3] = ex2_fast(fmaf(__uint_as_float(sv[e4 * 4 + 3]), a.scale_log2e, -l4.w));
                    }
                } else {
                    const bool diag = (i == j);
                    #pragma unroll
                    for (int e4 = 0; e4 < 8; e4++) {
                        const float4 l4 = *reinterpret_cast<const float4*>(stat + h2 * 32 + e4 * 4);
                        const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
                        #pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const int e = h2 * 32 + e4 * 4 + k;
                            float v = ex2_fast(fmaf(__uint_as_float(sv[e4 * 4 + k]), a.scale_log2e, -lv[k]));
                            if (diag && hf * 64 + e < r) v = 0.f;
                            p[e] = row_ok ? v : 0.f;
                        }
                    }
                }
            }
            {
                uint32_t pk[32];
                #pragma unroll
                for (int e = 0; e < 32; e++) pk[e] = pack_bf16x2(p[2 * e], p[2 * e + 1]);
                tmem_st16(tP + lane_off + hf * 32, pk);
                tmem_st16(tP + lane_off + hf * 32 + 16, pk + 16);
            }
            if (threadIdx.x == 128) TRACE(1, 2);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            if (threadIdx.x == 128) TRACE(1, 3);
            // ---- dS^T = P^T * (dP^T * scale - delta * scale), in four chunks of 16 queries: bf16 to TMEM (inside this half's own
            //      columns of the dP^T tile: a chunk's bf16 lands on fp32 columns that are already in registers) and to shared memory
            ok = mbar_wait(dp_full, t & 1, abort_flag, a.status, 0x6a3) && ok;
            if (t > 0) ok = mbar_wait(ds_empty, (t - 1) & 1, abort_flag, a.status, 0x6a4) && ok;     // dK / dQ (t-1) have read dS^T(t-1)
            tc_fence_after();
            if (threadIdx.x == 128) TRACE(1, 4);
            uint8_t* drow = sdS + hf * (BT * 128) + r * 128;
            #pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t dv[16];
                tmem_ld16(tdP + lane_off + hf * 64 + c * 16, dv);
                tmem_ld_wait();
                uint32_t dd[8];
                #pragma unroll
                for (int e4 = 0; e4 < 4; e4++) {
                    const float4 d4 = *reinterpret_cast<const float4*>(stat + BT + c * 16 + e4 * 4);
                    const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
                    float ds[4];
                    #pragma unroll
                    for (int k = 0; k < 4; k++) ds[k] = p[c * 16 + e4 * 4 + k] * fmaf(__uint_as_float(dv[e4 * 4 + k]), a.scale, -dl[k]);
                    dd[e4 * 2] = pack_bf16x2(ds[0], ds[1]);
                    dd[e4 * 2 + 1] = pack_bf16x2(ds[2], ds[3]);
                }
                tmem_st8(tdP + lane_off + hf * 64 + c * 8, dd);
                // 16 queries = 32 bytes = two 16-byte units 2c, 2c+1 of this row, 128-byte swizzle
                *reinterpret_cast<uint4*>(drow + (((2 * c) ^ (r & 7)) * 16)) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
                *reinterpret_cast<uint4*>(drow + (((2 * c + 1) ^ (r & 7)) * 16)) = make_uint4(dd[4], dd[5], dd[6], dd[7]);
            }
            tmem_st_wait();
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(ds_ready); mbar_arrive(&st_empty[t & 1]); }
            if (threadIdx.x == 128) TRACE(1, 5);
        }
    } else if (warp >= 12) {
        // ---------------------------------------------------------------- drain warps (128 threads): thread = row rr of a tile
        const int q = warp & 3;
        const int rr = q * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const float log2e = 1.4426950408889634f;
        const bool issuer = warp == 12 && lane == 0;
        bool ok = true;
        bool staged = false;
        uint32_t t = 0;
        int kvt = 0;
        // statistics of query rr of a pair's query tile -> table (tt & 1): LSE in log2 units, delta pre-multiplied by the scale;
        // queries past the end of the sequence get LSE = +inf, so that their P^T column is zero
        auto put_stats = [&](const Walk& pr, uint32_t tt) {
            const int tq = pr.i * BT + rr;
            float l = INFINITY, d = 0.f;
            if (tq < a.T) { l = a.lse[(size_t)pr.bh * a.T + tq] * log2e; d = a.delta[(size_t)pr.bh * a.T + tq] * a.scale; }
            ok = mbar_wait_relaxed(&st_empty[tt & 1], ((tt >> 1) & 1) ^ 1, abort_flag, a.status, 0x6b0) && ok;
            float* tab = sStat + (tt & 1) * (2 * BT);
            tab[rr] = l; tab[BT + rr] = d;
            __syncwarp();
            if (lane == 0) mbar_arrive(&st_full[tt & 1]);
        };
        if (wk.valid()) put_stats(wk, 0);
        for (; wk.valid(); t++) {
            const int bh = wk.bh, b = wk.b, h = wk.h, i = wk.i, j = wk.j;
            const bool last = wk.last_of_tile();
            wk.next();
            if (wk.valid()) put_stats(wk, t + 1);        // the next pair's table, one pair ahead
            // ---- the pair's dQ contribution: 64 fp32 of query row rr, slot order [group of 4 columns][row][4 floats],
            if (threadIdx.x == 384) TRACE(2, 0);
            ok = mbar_wait_relaxed(dq_full, t & 1, abort_flag, a.status, 0x6b1) && ok;
            tc_fence_after();
            if (threadIdx.x == 384) TRACE(2, 1);
            // through the staging buffer and one bulk copy: 16 global stores per thread and pair through the load/store unit held up
            // the shared-memory reads of the softmax warps for about a thousand cycles per pair (measured)
            float* slot = a.dq_ws + ((size_t)bh * npairs + (size_t)(i * (i + 1) / 2 + j)) * SLOT_FLOATS;
            if (staged) { if (issuer) tma_store_wait_read<0>(); asm volatile("bar.sync 1, 128;" ::: "memory"); }      // the previous copy has read the buffer
            #pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tmem_ld32(tdQ + lane_off + c * 32, v);
                tmem_ld_wait();
                if (c == 1) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(dq_empty); }
                #pragma unroll
                for (int e = 0; e < 8; e++)
                    *reinterpret_cast<uint4*>(sOut + (c * 8 + e) * (BT * 16) + rr * 16) = make_uint4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
            }
            fence_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (issuer && ok) {
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(slot), "r"(smem_u32(sOut)), "r"(SLOT_FLOATS * 4) : "memory");
                tma_store_commit();
            }
            staged = true;
            if (threadIdx.x == 384) TRACE(2, 2);
            if (last) {
                // ---- end of a key tile: dV_j and dK_j as bf16 tiles in the layout of a 128-byte-swizzled TMA box, one bulk store
                //      each (rows past T are clipped by TMA); a warp writing rows itself would touch 32 cache lines per instruction
                ok = mbar_wait_relaxed(acc_full, kvt & 1, abort_flag, a.status, 0x6b2) && ok;
                tc_fence_after();
                if (staged) { if (issuer) tma_store_wait_read<0>(); asm volatile("bar.sync 1, 128;" ::: "memory"); }
                #pragma unroll
                for (int which = 0; which < 2; which++) {
                    uint8_t* orow = sOut + which * TILE_BYTES + rr * 128;
                    #pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint32_t v[32];
                        tmem_ld32((which == 0 ? tdV : tdK) + lane_off + c * 32, v);
                        tmem_ld_wait();
                        #pragma unroll
                        for (int u = 0; u < 4; u++) {
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(v[8 * u]), __uint_as_float(v[8 * u + 1]));
                            o.y = pack_bf16x2(__uint_as_float(v[8 * u + 2]), __uint_as_float(v[8 * u + 3]));
                            o.z = pack_bf16x2(__uint_as_float(v[8 * u + 4]), __uint_as_float(v[8 * u + 5]));
                            o.w = pack_bf16x2(__uint_as_float(v[8 * u + 6]), __uint_as_float(v[8 * u + 7]));
                            *reinterpret_cast<uint4*>(orow + (((c * 4 + u) ^ (rr & 7)) * 16)) = o;
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty);
                fence_async_smem();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (issuer && ok) {
                    tma_store_4d(&tmDQKV, sOut, 0, 2 * a.NH + h, j * BT, b);
                    tma_store_4d(&tmDQKV, sOut + TILE_BYTES, 0, a.NH + h, j * BT, b);
                    tma_store_commit();
                }
                staged = true;
                kvt++;
            }
        }
        if (issuer) tma_store_wait<0>();
    }
#undef TRACE
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {
        long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// dQ[b, t, h, :] = bf16( sum over j = 0..i of slot(j, i)[r, :] ), i = t / 128, r = t % 128, added in the order of j.
// One CTA per (batch, head, query tile), heaviest tiles first.  A slot is read as it was written (order [group of 4 columns][row]
// [4 floats]): a warp reads 512 contiguous bytes per instruction, every thread has 16 loads of 16 bytes in flight (two slots);
// the sums are transposed through shared memory so that the 8 lanes of a row store its 128 bytes together.
__global__ void __launch_bounds__(256)
dq_fold_kernel(bf16* __restrict__ dqkv, const float* __restrict__ ws, int B, int T, int NH, int nt) {
    __shared__ __align__(16) bf16 tile[BT][HS + 8];
    const int nbh = B * NH;
    const int i = nt - 1 - (int)(blockIdx.x / nbh);
    const int bh = (int)(blockIdx.x % nbh);
    const int npairs = nt * (nt + 1) / 2;
    const int t = threadIdx.x;
    const float* src = ws + ((size_t)bh * npairs + (size_t)(i * (i + 1) / 2)) * SLOT_FLOATS + t * 4;
    f32x4 acc[8];
    #pragma unroll
    for (int k = 0; k < 8; k++)
        #pragma unroll
        for (int e = 0; e < 4; e++) acc[k][e] = 0.f;
    for (int j = 0; j <= i; j += 2) {
        const bool two = j + 1 <= i;
        f32x4 a0[8], a1[8];
        #pragma unroll
        for (int k = 0; k < 8; k++) a0[k] = ld128cs(src + (size_t)j * SLOT_FLOATS + k * 1024);
        if (two) {
            #pragma unroll
            for (int k = 0; k < 8; k++) a1[k] = ld128cs(src + (size_t)(j + 1) * SLOT_FLOATS + k * 1024);
        }
        #pragma unroll
        for (int k = 0; k < 8; k++)
            #pragma unroll
            for (int e = 0; e < 4; e++) acc[k][e] += a0[k][e];
        if (two) {
            #pragma unroll
            for (int k = 0; k < 8; k++)
                #pragma unroll
                for (int e = 0; e < 4; e++) acc[k][e] += a1[k][e];
        }
    }
    // thread t holds row t % 128, column groups 2k + t / 128
    const int row = t & (BT - 1), g0 = t >> 7;
    #pragma unroll
    for (int k = 0; k < 8; k++) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[k][0], acc[k][1]), hi = __floats2bfloat162_rn(acc[k][2], acc[k][3]);
        uint2 w;
        w.x = *reinterpret_cast<uint32_t*>(&lo);
        w.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(&tile[row][(2 * k + g0) * 4]) = w;
    }
    __syncthreads();
    const int b = bh / NH, h = bh - b * NH;
    #pragma unroll
    for (int q = 0; q < 4; q++) {
        const int c = q * 256 + t, r = c >> 3, c8 = c & 7;
        const int tq = i * BT + r;
        if (tq < T)
            *reinterpret_cast<uint4*>(dqkv + (((size_t)b * T + tq) * 3) * NH * HS + (size_t)h * HS + c8 * 8) = *reinterpret_cast<const uint4*>(&tile[r][c8 * 8]);
    }
}

}  // namespace

// Profiling aid: with a device buffer of 4 * 8 * 64 int64 set here, CTA 0 of every later single-pass launch records clock64()
// stamps of its first 64 tile pairs (role 0 = issuer, 1 = first softmax warp, 2 = first drain warp; events in program
// order).  Null (the default) switches it off.
static long long* g_trace = nullptr;
extern "C" int llmc_attention_bwd_set_trace(long long* buf) { g_trace = buf; return 0; }

// number of fp32 words of workspace that llmc_attention_bwd needs (delta + the dQ contributions of the single-pass kernel)
extern "C" long long llmc_attention_bwd_workspace(int B, int T, int NH, int hs) {
    long long words = (long long)B * NH * T;                       // delta
    words = (words + 63) & ~63ll;
    if (hs == HS) {
        const long long nt = CEIL_DIV(T, BT);
        words += (long long)B * NH * (nt * (nt + 1) / 2) * SLOT_FLOATS;
    }
    return words;
}

// dqkv (B,T,3,NH,HS) = gradient of causal attention; ws: llmc_attention_bwd_workspace(...) floats.  Head sizes: multiples of 8, 64..128.
extern "C" int llmc_attention_bwd(bf16* dqkv, float* ws, const bf16* dout, const bf16* qkv, const bf16* out, const float* lse,
                                  int B, int T, int NH, int hs, cudaStream_t stream) {
    if (hs != HS) return llmc_attention_bwd_two_pass(dqkv, ws, dout, qkv, out, lse, B, T, NH, hs, stream);
    if ((reinterpret_cast<uintptr_t>(ws) & 15u) != 0) return -1;
    float* delta = ws;
    float* dq_ws = ws + ((((long long)B * NH * T) + 63) & ~63ll);
    CUtensorMap tmQKV, tmDO, tmDQKV;
    int rc = llmc_attn_qkv_map(&tmQKV, qkv, B, T, NH, hs);
    if (rc) return rc;
    {
        uint64_t dims[4] = {(uint64_t)hs, (uint64_t)NH, (uint64_t)T, (uint64_t)B};
        uint64_t strides[4] = {2, (uint64_t)hs * 2, (uint64_t)NH * hs * 2, (uint64_t)T * NH * hs * 2};
        uint32_t box[4] = {64, 1, 128, 1};
        if ((rc = llmc_get_tensormap(&tmDO, dout, 2, 4, dims, strides, box, 3))) return rc;
    }
    if ((rc = llmc_attn_qkv_map(&tmDQKV, dqkv, B, T, NH, hs))) return rc;
    if ((rc = llmc_attention_delta(delta, out, dout, B, T, NH, hs, stream))) return rc;
    Args a;
    a.dqkv = dqkv; a.dq_ws = dq_ws; a.lse = lse; a.delta = delta; a.B = B; a.T = T; a.NH = NH;
    a.scale = 1.0f / sqrtf((float)hs);
    a.scale_log2e = a.scale * 1.4426950408889634f;
    a.status = llmc_status_ptr();
    a.trace = g_trace;
    const int nt = CEIL_DIV(T, BT);
    const int total = B * NH * ((nt + 1) / 2);
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int grid = total < sms ? total : sms;
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(attn_bwd1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        configured = true;
    }
    attn_bwd1_kernel<<<grid, THREADS, SMEM, stream>>>(tmQKV, tmDO, tmDQKV, a);
    CUDA_CHECK(cudaGetLastError());
    dq_fold_kernel<<<(unsigned)(B * NH * nt), 256, 0, stream>>>(dqkv, dq_ws, B, T, NH, nt);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
