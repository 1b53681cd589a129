// Causal flash attention forward for sm_100a, head size 64, on the packed (B, T, 3, NH, HS) QKV layout.
//
// A CTA works on TWO adjacent 128-row query tiles (A = 2p, B = 2p + 1) of one (batch, head) at a time and streams the key /
// value tiles 0..2p+1 past both (B takes one tile more than A), so every K / V tile is loaded once for 256 queries.
//
//   warp 0       TMA producer: the two Q tiles of an item (double buffered across items), then K_j, V_j through a 3-stage ring.
//   warp 1       issuer of S_X = Q_X K_j^T (SS) and O_X += P_X V_j (TS: A = P_X in tensor memory), X in {A, B}; the warp runs in
//                uniform control flow with one elected lane executing the tcgen05 instructions.
//   warps 4-7    softmax of tile A, warps 8-11 softmax of tile B: ONE THREAD PER QUERY ROW holding the row's 128 scores in
//                registers.  Row maximum and row sum need no exchange between threads; P goes back to tensor memory as bf16
//                (no shared-memory round trip, no proxy fence); O accumulates in tensor memory across the key tiles and is
//                rescaled by its own row's thread only when the running maximum grows by more than 2^8 (the stale maximum
//                is a valid reference point for the exponentials in between, the final division by the row sum cancels it).
//                The two groups are half a tile out of phase: one group's exponentials run under the other's products.
//
// TMEM columns: S_A [0,128)  S_B [128,256)  O_A [256,320)  O_B [320,384)  P_A [384,448)  P_B [448,512)   (P: 128 bf16 per row)
//
// Statistics are written as natural-log LSE per (b, h, t), the layout cuDNN's SDPA uses in the reference
// (llmc/cudnn_att.cpp:105-113).  Output tiles leave through shared memory and TMA stores (rows past T are clipped).
// Head sizes above 64 use the kernel of attention_fwd.cu.
//
// Capability parity: attention_forward_cudnn (llmc/cudnn_att.cpp:222-254) and attention_forward of llmc/attention.cuh.
#include "common.cuh"

int llmc_attn_qkv_map(CUtensorMap* tm, const bf16* qkv, int B, int T, int NH, int hs);   // attention_fwd.cu
int llmc_attention_fwd_general(bf16* out, float* lse, const bf16* qkv, int B, int T, int NH, int hs, cudaStream_t stream);

namespace {

constexpr int BT = 128;
constexpr int HS = 64;
constexpr int TILE_BYTES = BT * HS * 2;             // 16 KB: one 128-byte-swizzled TMA box
constexpr int QBUF = 2;                             // Q pair buffers (current / next item)
constexpr int KVSTAGES = 3;
constexpr int THREADS = 384;                        // TMA warp, issuer warp, two idle warps, 2 x 4 softmax warps
constexpr int TMEM_COLS = 512;
constexpr int SMEM = QBUF * 2 * TILE_BYTES + KVSTAGES * 2 * TILE_BYTES + 2 * TILE_BYTES + 256;      // Q, K/V ring, two output tiles
constexpr long long SKEW_CYCLES = 1200;
constexpr float RESCALE_LOG2 = 8.0f;                // the running maximum may lag by this much (in log2 units of the scaled scores)

struct Args {
    float* lse;        // (B, NH, T)
    int B, T, NH;
    float scale_log2e; // (1/sqrt(HS)) * log2(e)
    float scale;
    unsigned int* status;
    long long* trace;  // optional: [3 roles][8 events][64 tiles] clock64() stamps of CTA 0 (null in normal runs)
};
#define TRACE(role, ev, tt) do { if (a.trace != nullptr && blockIdx.x == 0 && (tt) < 64) a.trace[((role) * 8 + (ev)) * 64 + (tt)] = clock64(); } while (0)

DEVINL void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attn_fwd1_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmOut, const Args a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                                   // [QBUF][A, B]
    uint8_t* sK = sQ + QBUF * 2 * TILE_BYTES;             // [KVSTAGES]
    uint8_t* sV = sK + KVSTAGES * TILE_BYTES;             // [KVSTAGES]
    uint8_t* sO = sV + KVSTAGES * TILE_BYTES;             // [A, B] output tiles on their way out
    uint64_t* bars = reinterpret_cast<uint64_t*>(sO + 2 * TILE_BYTES);
    uint64_t* q_full = bars + 0;      // [2]
    uint64_t* q_empty = bars + 2;     // [2]
    uint64_t* k_full = bars + 4;      // [3]
    uint64_t* k_empty = bars + 7;     // [3]
    uint64_t* v_full = bars + 10;     // [3]
    uint64_t* v_empty = bars + 13;    // [3]
    uint64_t* s_full = bars + 16;     // [2 slots] S_X(t) complete                            (1 commit)
    uint64_t* s_empty = bars + 18;    // [2] the slot's warps hold S_X(t) in registers          (4 arrivals)
    uint64_t* p_ready = bars + 20;    // [2] P_X(t) is in TMEM (and O_X rescaled if needed)     (4 arrivals)
    uint64_t* pv_done = bars + 22;    // [2] O_X += P_X(t) V complete                           (1 commit)
    uint64_t* o_free = bars + 24;     // [2] the slot's warps hold the item's O_X in registers  (4 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nq = CEIL_DIV(a.T, BT);
    const int np = (nq + 1) >> 1;                         // query-tile pairs per (batch, head)
    const int BH = a.B * a.NH;
    const int total = BH * np;
    // work item w -> (pair p, batch, head); late (heavy) pairs first
    auto decode = [&](int w, int& p, int& b, int& h) {
        const int rank = w / BH, bh = w - rank * BH;
        p = np - 1 - rank;
        b = bh / a.NH; h = bh - b * a.NH;
    };

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) record_error(a.status, ST_BAD_ARG, 0x18);
        for (int i = 0; i < 2; i++) {
            mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&p_ready[i], 4); mbar_init(&pv_done[i], 1); mbar_init(&o_free[i], 4);
        }
        for (int i = 0; i < KVSTAGES; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmOut);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int kst = 0; uint32_t kph = 0;
            int it = 0;
            bool fail = false;
            for (int w = blockIdx.x; w < total && !fail; w += gridDim.x, it++) {
                int p, b, h; decode(w, p, b, h);
                const int qb = it & 1;
                if (!mbar_wait_relaxed(&q_empty[qb], ((it >> 1) & 1) ^ 1, abort_flag, a.status, 0x502)) break;
                mbar_expect_tx(&q_full[qb], 2 * TILE_BYTES);
                tma_load_4d(sQ + qb * 2 * TILE_BYTES, &tmQKV, &q_full[qb], 0, h, 2 * p * BT, b);                       // Q_A
                tma_load_4d(sQ + qb * 2 * TILE_BYTES + TILE_BYTES, &tmQKV, &q_full[qb], 0, h, (2 * p + 1) * BT, b);    // Q_B (zeros past T)
                const int nkv = min(2 * p + 2, nq);
                for (int j = 0; j < nkv; j++) {
                    if (!mbar_wait_relaxed(&k_empty[kst], kph ^ 1, abort_flag, a.status, 0x500)) { fail = true; break; }
                    mbar_expect_tx(&k_full[kst], TILE_BYTES);
                    tma_load_4d(sK + kst * TILE_BYTES, &tmQKV, &k_full[kst], 0, a.NH + h, j * BT, b);
                    if (!mbar_wait_relaxed(&v_empty[kst], kph ^ 1, abort_flag, a.status, 0x501)) { fail = true; break; }
                    mbar_expect_tx(&v_full[kst], TILE_BYTES);
                    tma_load_4d(sV + kst * TILE_BYTES, &tmQKV, &v_full[kst], 0, 2 * a.NH + h, j * BT, b);
                    if (++kst == KVSTAGES) { kst = 0; kph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- issuer
        // Per item and key tile j, in this order:  S_A(j+1),  S_B(j+1),  O_A += P_A(j) V_j,  O_B += P_B(j) V_j;  tile A stops one
        // key tile before tile B.  The first S of the next item is issued at the end of the current one.
        const bool leader = elect_one();
#define WAIT_ALL(bar, parity, code) (__all_sync(0xffffffffu, mbar_wait_relaxed(bar, parity, abort_flag, a.status, code)) != 0)
        constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BT, 0, 0);      // Q (K-major) x K (K-major)
        constexpr uint32_t idesc_o = umma_idesc_bf16(BT, HS, 0, 1);      // P (TMEM) x V (N-major)
        constexpr uint32_t TILE_UNITS = TILE_BYTES / 16;
        const uint64_t dQ0 = umma_desc_sw128(smem_u32(sQ), 16, 1024), dK0 = umma_desc_sw128(smem_u32(sK), 16, 1024);
        const uint64_t dV0 = umma_desc_sw128(smem_u32(sV), TILE_BYTES, 1024);
        uint32_t ts[2] = {0, 0};          // tiles issued per slot (S products), for the parities of s_empty
        uint32_t tp[2] = {0, 0};          // tiles whose P V product has been issued per slot
        uint32_t items[2] = {0, 0};       // items started per slot, for o_free
        int kst = 0; uint32_t kph = 0;    // ring position of key tile j of the current item
        bool ok = true;
        // S_X of the key tile at ring stage st with the Q tile of buffer qb; the slot that reads a K tile (a Q pair) last releases it
        auto issue_s = [&](int x, int qb, int st, bool release_k, bool release_q) {
            const uint64_t q = dQ0 + (uint32_t)(qb * 2 + x) * TILE_UNITS, k = dK0 + (uint32_t)st * TILE_UNITS;
            if (leader) {
                #pragma unroll
                for (int kk = 0; kk < HS / 16; kk++) umma_ss(tmem_base + x * 128, q + 2 * kk, k + 2 * kk, idesc_s, kk > 0);
                umma_commit(&s_full[x]);
                TRACE(0, x * 2 + 1, ts[x]);
                if (release_k) umma_commit(&k_empty[st]);
                if (release_q) umma_commit(&q_empty[qb]);
            }
            ts[x]++;
        };
        // first S products of an item (key tile 0 at stage st): slot A, and slot B if the item has a second query tile
        auto issue_first = [&](int p_, int qb, int st) {
            const bool hb = 2 * p_ + 1 < nq;
            issue_s(0, qb, st, !hb, !hb && p_ == 0);
            if (hb) issue_s(1, qb, st, true, false);
        };
        // O_X += P_X(jj) V_jj : A = P_X in TMEM (16 keys = 8 columns per step), B = V_jj N-major (16 rows = 2048 bytes)
        auto issue_pv = [&](int x, int jj, int st, uint32_t ph, bool release_v) {
            bool good = WAIT_ALL(&v_full[st], ph, 0x515) && WAIT_ALL(&p_ready[x], tp[x] & 1, 0x514);
            if (good && jj == 0 && items[x] > 0) good = WAIT_ALL(&o_free[x], (items[x] - 1) & 1, 0x517);
            if (!good) return false;
            tc_fence_after();
            const uint64_t v = dV0 + (uint32_t)st * TILE_UNITS;
            if (leader) {
                #pragma unroll
                for (int kk = 0; kk < BT / 16; kk++)
                    umma_ts(tmem_base + 256 + x * 64, tmem_base + 384 + x * 64 + kk * 8, v + 128 * kk, idesc_o, (jj > 0 || kk > 0));
                umma_commit(&pv_done[x]);
                if (release_v) umma_commit(&v_empty[st]);
                TRACE(0, x * 2, tp[x]);
            }
            tp[x]++;
            if (jj == 0) items[x]++;
            return true;
        };
        int it = 0;
        uint32_t kabs = 0;                // key tiles of earlier items: tile jj of the current item sits at ring position kabs + jj
        if ((int)blockIdx.x < total) {
            int p, b, h; decode(blockIdx.x, p, b, h);
            ok = WAIT_ALL(&q_full[0], 0, 0x510) && WAIT_ALL(&k_full[0], 0, 0x511);
            tc_fence_after();
            if (ok) issue_first(p, 0, 0);
        }
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x, it++) {
            int p, b, h; decode(w, p, b, h);
            const int qb = it & 1;
            const bool hasB = 2 * p + 1 < nq;
            const int nA = 2 * p + 1, nB = hasB ? 2 * p + 2 : 0;
            const int nkv = hasB ? nB : nA;
            bool next_item = false; int np_ = 0;
            if (w + (int)gridDim.x < total) { int b2, h2; decode(w + gridDim.x, np_, b2, h2); next_item = true; }
            // The order inside a step is the order in which the events arrive when slot B runs half a tile behind slot A:
            //   S_A(j+1) [A holds S_A(j)],  O_B += P_B(j-1) V,  S_B(j+1) [B holds S_B(j)],  O_A += P_A(j) V.
            // With this order a lagging slot B never holds up slot A, so the skew (see the softmax warps) survives.
            for (int j = 0; j <= nkv && ok; j++) {
                const uint32_t pos = kabs + j;
                const int st_prev = (pos + KVSTAGES - 1) % KVSTAGES, st_cur = pos % KVSTAGES, st_next = (pos + 1) % KVSTAGES;
                const uint32_t ph_prev = ((pos - 1) / KVSTAGES) & 1, ph_cur = (pos / KVSTAGES) & 1, ph_next = ((pos + 1) / KVSTAGES) & 1;
                if (j + 1 < nkv) ok = WAIT_ALL(&k_full[st_next], ph_next, 0x512);
                if (ok && j + 1 < nA) {
                    ok = WAIT_ALL(&s_empty[0], (ts[0] - 1) & 1, 0x513);
                    if (ok) { tc_fence_after(); issue_s(0, qb, st_next, !hasB, !hasB && j + 1 == nA - 1); }
                }
                if (ok && j >= 1 && j - 1 < nB) ok = issue_pv(1, j - 1, st_prev, ph_prev, true);
                if (ok && j + 1 < nB) {
                    ok = WAIT_ALL(&s_empty[1], (ts[1] - 1) & 1, 0x513);
                    if (ok) { tc_fence_after(); issue_s(1, qb, st_next, true, j + 1 == nB - 1); }
                }
                // ---- first S products of the next item, once both slots hold their last S of this one
                if (ok && next_item && j == nkv - 1) {
                    ok = WAIT_ALL(&q_full[qb ^ 1], ((it + 1) >> 1) & 1, 0x516) && WAIT_ALL(&k_full[(kabs + nkv) % KVSTAGES], ((kabs + nkv) / KVSTAGES) & 1, 0x51a);
                    if (ok && ts[0] > 0) ok = WAIT_ALL(&s_empty[0], (ts[0] - 1) & 1, 0x518);
                    if (ok && ts[1] > 0 && 2 * np_ + 1 < nq) ok = WAIT_ALL(&s_empty[1], (ts[1] - 1) & 1, 0x519);
                    if (ok) { tc_fence_after(); issue_first(np_, qb ^ 1, (kabs + nkv) % KVSTAGES); }
                }
                if (ok && j < nA) ok = issue_pv(0, j, st_cur, ph_cur, !hasB);
            }
            kabs += nkv;
        }
#undef WAIT_ALL
    }
    else if (warp >= 4) {
        // ---------------------------------------------------------------- softmax of slot x: thread = query row r of the slot's tile
        const int x = (warp - 4) >> 2;
        const int q4 = warp & 3;
        const int r = q4 * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
        const uint32_t tS = tmem_base + x * 128, tO = tmem_base + 256 + x * 64, tP = tmem_base + 384 + x * 64;
        const bool issuer = q4 == 0 && lane == 0;          // the thread of the slot that issues its output store
        const float c = a.scale_log2e;
        bool ok = true;
        bool staged = false;
        uint32_t t = 0;                                    // tiles of this slot so far
        int it = 0;
        for (int w = blockIdx.x; w < total; w += gridDim.x, it++) {
            int p, b, h; decode(w, p, b, h);
            const int qi = 2 * p + x;                      // this slot's query tile
            if (qi >= nq) continue;                        // (uniform for the slot) no second tile in this item
            float m = -INFINITY, l = 0.f;                  // reference maximum (raw score units) and row sum relative to it
            // The two slots share the special-function unit: started together (their first S products are issued together) they
            // would run their exponentials at the same time, at half rate each, and their loads, maxima and waits at the same
            // time, with the unit idle.  Half a tile of skew (slot B pauses once its first S of the item is there) puts one slot's
            // exponentials under the other's remaining work.
            for (int j = 0; j <= qi; j++, t++) {
                if (r == 0) TRACE(1 + x, 0, t);
                ok = mbar_wait(&s_full[x], t & 1, abort_flag, a.status, 0x520 + x) && ok;
                if (x == 1 && j == 0) { const long long t0 = clock64(); while (clock64() - t0 < SKEW_CYCLES) { } }
                tc_fence_after();
                if (r == 0) TRACE(1 + x, 1, t);
                uint32_t sv[128];
                tmem_ld32(tS + lane_off, sv);
                tmem_ld32(tS + lane_off + 32, sv + 32);
                tmem_ld32(tS + lane_off + 64, sv + 64);
                tmem_ld32(tS + lane_off + 96, sv + 96);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[x]);       // S_X of the next key tile may be issued
                if (r == 0) TRACE(1 + x, 2, t);
                if (j == qi) {
                    #pragma unroll
                    for (int e = 0; e < 128; e++) if (e > r) sv[e] = 0xff800000u;      // -inf above the diagonal
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
                #pragma unroll
                for (int e = 0; e < 128; e += 4) {
                    mx0 = fmaxf(mx0, __uint_as_float(sv[e])); mx1 = fmaxf(mx1, __uint_as_float(sv[e + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(sv[e + 2])); mx3 = fmaxf(mx3, __uint_as_float(sv[e + 3]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                // move the reference maximum only when it lags by more than 2^RESCALE_LOG2 (decided per warp, so that the
                // TMEM accesses stay warp-wide); a moved maximum rescales the row sum now and the row of O_X below
                const bool grow = (mx - m) * c > RESCALE_LOG2 || j == 0;
                const bool moved = __any_sync(0xffffffffu, grow) != 0;
                float alpha = 1.0f;
                if (moved) {
                    const float m_new = fmaxf(m, mx);
                    alpha = ex2_fast((m - m_new) * c);      // 0 on the first tile (m = -inf)
                    l *= alpha;
                    m = m_new;
                }
                if (r == 0) TRACE(1 + x, 3, t);
                const float moff = m * c;
                float rs0 = 0.f, rs1 = 0.f;
                uint32_t pk[64];
                #pragma unroll
                for (int e = 0; e < 128; e += 2) {
                    const float p0 = ex2_fast(fmaf(__uint_as_float(sv[e]), c, -moff));
                    const float p1 = ex2_fast(fmaf(__uint_as_float(sv[e + 1]), c, -moff));
                    rs0 += p0; rs1 += p1;
                    pk[e >> 1] = pack_bf16x2(p0, p1);
                }
                l += rs0 + rs1;
                if (r == 0) TRACE(1 + x, 5, t);
                // the previous product has read P_X(t-1) and finished adding to O_X: only now is it waited for, so that it ran
                // under the exponentials above
                if (j > 0) ok = mbar_wait(&pv_done[x], (t - 1) & 1, abort_flag, a.status, 0x524 + x) && ok;
                tc_fence_after();
                if (r == 0) TRACE(1 + x, 4, t);
                if (moved && j > 0) {
                    #pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t ov[32];
                        tmem_ld32(tO + lane_off + half * 32, ov);
                        tmem_ld_wait();
                        #pragma unroll
                        for (int e = 0; e < 32; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
                        tmem_st16(tO + lane_off + half * 32, ov);
                        tmem_st16(tO + lane_off + half * 32 + 16, ov + 16);
                    }
                }
                tmem_st16(tP + lane_off, pk);
                tmem_st16(tP + lane_off + 16, pk + 16);
                tmem_st16(tP + lane_off + 32, pk + 32);
                tmem_st16(tP + lane_off + 48, pk + 48);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[x]);
                if (r == 0) TRACE(1 + x, 6, t);
            }
            // ---- item epilogue: O_X / l -> bf16 tile in the layout of a 128-byte-swizzled TMA box -> one bulk store
            ok = mbar_wait(&pv_done[x], (t - 1) & 1, abort_flag, a.status, 0x528 + x) && ok;
            tc_fence_after();
            if (staged) { if (issuer) tma_store_wait_read<0>(); asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory"); }
            const float inv = 1.0f / l;
            uint8_t* orow = sO + x * TILE_BYTES + r * 128;
            #pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t ov[32];
                tmem_ld32(tO + lane_off + half * 32, ov);
                tmem_ld_wait();
                #pragma unroll
                for (int u = 0; u < 4; u++) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(ov[8 * u]) * inv, __uint_as_float(ov[8 * u + 1]) * inv);
                    o.y = pack_bf16x2(__uint_as_float(ov[8 * u + 2]) * inv, __uint_as_float(ov[8 * u + 3]) * inv);
                    o.z = pack_bf16x2(__uint_as_float(ov[8 * u + 4]) * inv, __uint_as_float(ov[8 * u + 5]) * inv);
                    o.w = pack_bf16x2(__uint_as_float(ov[8 * u + 6]) * inv, __uint_as_float(ov[8 * u + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + (((half * 4 + u) ^ (r & 7)) * 16)) = o;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[x]);            // O_X may be overwritten by the next item's first product
            fence_async_smem();
            asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");
            if (issuer && ok) {
                tma_store_4d(&tmOut, sO + x * TILE_BYTES, 0, h, qi * BT, b);
                tma_store_commit();
            }
            staged = true;
            const int trow = qi * BT + r;
            if (trow < a.T && ok) a.lse[((size_t)b * a.NH + h) * a.T + trow] = m * a.scale + logf(l);
        }
        if (issuer) tma_store_wait<0>();
    }
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

#undef TRACE
}  // namespace

// Profiling aid: with a device buffer of 3 * 8 * 64 int64 set here, CTA 0 of every later launch records clock64() stamps of its
// first 64 tiles per slot (role 0 = issuer, 1 / 2 = first thread of the softmax group of tile A / B).  Null switches it off.
static long long* g_fwd_trace = nullptr;
extern "C" int llmc_attention_fwd_set_trace(long long* buf) { g_fwd_trace = buf; return 0; }

// out (B,T,NH,HS) = causal softmax(Q K^T / sqrt(HS)) V ; lse (B,NH,T) fp32.  Head sizes: multiples of 8 from 64 to 128.
extern "C" int llmc_attention_fwd(bf16* out, float* lse, const bf16* qkv, int B, int T, int NH, int hs, cudaStream_t stream) {
    if (hs != HS) return llmc_attention_fwd_general(out, lse, qkv, B, T, NH, hs, stream);
    CUtensorMap tmQKV, tmOut;
    int rc = llmc_attn_qkv_map(&tmQKV, qkv, B, T, NH, hs);
    if (rc) return rc;
    {
        uint64_t dims[4] = {(uint64_t)hs, (uint64_t)NH, (uint64_t)T, (uint64_t)B};
        uint64_t strides[4] = {2, (uint64_t)hs * 2, (uint64_t)NH * hs * 2, (uint64_t)T * NH * hs * 2};
        uint32_t box[4] = {64, 1, 128, 1};
        if ((rc = llmc_get_tensormap(&tmOut, out, 2, 4, dims, strides, box, 3))) return rc;
    }
    Args a;
    a.lse = lse; a.B = B; a.T = T; a.NH = NH;
    a.scale = 1.0f / sqrtf((float)hs);
    a.scale_log2e = a.scale * 1.4426950408889634f;
    a.status = llmc_status_ptr();
    a.trace = g_fwd_trace;
    const int nq = CEIL_DIV(T, BT);
    const int total = B * NH * ((nq + 1) / 2);
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int grid = total < sms ? total : sms;
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(attn_fwd1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        configured = true;
    }
    attn_fwd1_kernel<<<grid, THREADS, SMEM, stream>>>(tmQKV, tmOut, a);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
