// Causal flash attention backward for sm_100a on the packed (B, T, 3, NH, HS) layout; head sizes 64..128
// (multiples of 8; sizes above 64 run as a 128-wide head whose missing channels TMA fills with zeros).
//
// Deterministic by construction: no atomics, every output element has one writer and a fixed
// summation order.  Three launches:
//   1. delta[b,h,t] = sum_d O[b,t,h,d] * dO[b,t,h,d]
//   2. "dK/dV" kernel: one CTA per (b, h, 128-row key/value tile).  K_j and V_j stay resident in
//      shared memory while the query tiles i >= j stream through a 2-stage TMA ring.  Per query tile
//      S = Q K^T and dP = dO V^T are formed in TMEM, the 512 softmax threads turn them into
//      P = exp(S*scale - LSE) and dS = P (dP - delta) scale (bf16, swizzled shared memory), and
//      dV += P^T dO, dK += dS^T Q accumulate in TMEM over the whole loop (MN-major A operands).
//   3. "dQ" kernel: one CTA per (b, h, query tile); K_j, V_j stream; dQ += dS K accumulates in TMEM.
// S and dP are recomputed in (3) instead of exchanging dQ partials through atomics; that costs two
// extra MMAs per tile and buys bit-reproducible gradients, which the reference also demands of
// cuDNN (llmc/cudnn_att.cpp:186-191).
//
// Both MMA kernels are persistent (one CTA per SM walks a heavy-first list of work items; resident tiles and
// TMEM accumulators are double buffered across items).  A CTA has 608 threads: warp 0 TMA producer, warp 1 issuer of the score
// products (S, dP), warps 2..17 softmax/epilogue (thread = one row x one 32-column quarter), warp 18 issuer of the accumulating
// products (dV, dK or dQ).  The softmax threads pull S/dP into registers and release the TMEM tiles at once, so the next
// tile's S/dP MMAs run underneath the exponentials.
//
// Capability parity: attention_backward_cudnn (llmc/cudnn_att.cpp:256-288) and attention_backward
// of llmc/attention.cuh in the reference.
#include "common.cuh"

int llmc_attn_qkv_map(CUtensorMap* tm, const bf16* qkv, int B, int T, int NH, int hs);   // attention_fwd.cu

namespace {

constexpr int BT = 128;                             // tile rows (queries and keys)
constexpr int CHUNK_BYTES = 128 * 64 * 2;           // 16 KB: 128 rows x 64 channels, one 128-byte-swizzled TMA box
constexpr int PS_BYTES = BT * BT * 2;               // 32 KB
constexpr int BWD_THREADS = 608;                    // TMA warp + score-product issuer + 16 softmax warps + accumulate-product issuer
constexpr int BWD_TMEM_COLS = 512;

// NC = number of 64-channel chunks of the (zero-padded) head: 1 -> head size 64, 2 -> head sizes 72..128.
// With two chunks a tile pair is 64 KB and an accumulator pair fills the rest of TMEM, so that variant runs without
// double buffering (one resident buffer, one stream stage, one accumulator set).
template <int NC> struct BwdCfg {
    static constexpr int HSP = 64 * NC;
    static constexpr int TILE_BYTES = NC * CHUNK_BYTES;
    static constexpr int PAIR_BYTES = 2 * TILE_BYTES;
    static constexpr int RB = NC == 1 ? 2 : 1;          // resident pair buffers
    static constexpr int XSTAGES = NC == 1 ? 3 : 1;     // ring of streamed tile pairs
    static constexpr int ACCBUF = NC == 1 ? 2 : 1;      // TMEM accumulator sets (each 2 * HSP columns)
    static constexpr int SMEM = RB * PAIR_BYTES + XSTAGES * PAIR_BYTES + 2 * PS_BYTES + 256;
};

struct BwdArgs {
    bf16* dqkv;          // (B, T, 3, NH, HS)
    const float* lse;    // (B, NH, T)
    const float* delta;  // (B, NH, T)
    int B, T, NH, hs;
    float scale, scale_log2e;
    unsigned int* status;
};

__global__ void delta_kernel(float* __restrict__ delta, const bf16* __restrict__ out, const bf16* __restrict__ dout,
                             int B, int T, int NH, int hs) {
    // 8 lanes per (b, t, h) row of hs channels
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = gid >> 3;
    const int part = (int)(gid & 7);
    const long long rows = (long long)B * T * NH;
    float acc = 0.f;
    if (row < rows) {
        for (int p = part; p < (hs >> 3); p += 8) {
            bf16x8 o = ld128cs(out + row * hs + p * 8), d = ld128cs(dout + row * hs + p * 8);
            #pragma unroll
            for (int e = 0; e < 8; e++) acc += __bfloat162float(o[e]) * __bfloat162float(d[e]);
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (row < rows && part == 0) {
        const long long bt = row / NH; const int h = (int)(row % NH);
        const long long b = bt / T; const int t = (int)(bt % T);
        delta[(b * NH + h) * T + t] = acc;
    }
}

// DKV = true : resident (K_j, V_j), streamed (Q_i, dO_i), outputs dK_j, dV_j
// DKV = false: resident (Q_i, dO_i), streamed (K_j, V_j), output dQ_i
// Persistent: gridDim.x CTAs (one per SM) take work items w = blockIdx.x, blockIdx.x + gridDim.x, ...; the item list is
// ordered heavy first.  The resident pair and the TMEM accumulators are double buffered so that the loads and the first
// MMAs of the next item run underneath the epilogue of the current one.
template <bool DKV, int NC>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO, const BwdArgs a) {
    using Cfg = BwdCfg<NC>;
    constexpr int HSP = Cfg::HSP, TILE_BYTES = Cfg::TILE_BYTES, PAIR_BYTES = Cfg::PAIR_BYTES;
    constexpr int RB = Cfg::RB, XSTAGES = Cfg::XSTAGES, ACCBUF = Cfg::ACCBUF;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sRes = smem;                              // [RB][2 tiles]
    uint8_t* sStr = sRes + RB * PAIR_BYTES;            // [XSTAGES][2 tiles]
    uint8_t* sP = sStr + XSTAGES * PAIR_BYTES;
    uint8_t* sdS = sP + PS_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + PS_BYTES);
    uint64_t* res_full = bars + 0;    // [2]
    uint64_t* res_empty = bars + 2;   // [2]
    uint64_t* x_full = bars + 4;      // [XSTAGES]
    uint64_t* x_empty = bars + 8;     // [XSTAGES]
    uint64_t* sdp_full = bars + 12;
    uint64_t* sdp_empty = bars + 13;
    uint64_t* pds_full = bars + 14;
    uint64_t* pds_empty = bars + 15;
    uint64_t* acc_full = bars + 16;   // [2]
    uint64_t* acc_empty = bars + 18;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = CEIL_DIV(a.T, BT);
    const int BH = a.B * a.NH;
    const int total = BH * nt;
    // work item -> (fixed tile, batch, head, number of streamed tiles); heavy items first:
    // key tile 0 sees every query tile; query tile nt-1 sees every key tile
    auto decode = [&](int w, int& fixed, int& b, int& h, int& cnt) {
        const int rank = w / BH, bh = w - rank * BH;
        fixed = DKV ? rank : (nt - 1 - rank);
        cnt = DKV ? (nt - fixed) : (fixed + 1);
        b = bh / a.NH; h = bh - b * a.NH;
    };

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) record_error(a.status, ST_BAD_ARG, 0x20);
        for (int i = 0; i < 2; i++) {
            mbar_init(&res_full[i], 1); mbar_init(&res_empty[i], 1);
            mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 16);
        }
        for (int i = 0; i < XSTAGES; i++) { mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1); }
        mbar_init(sdp_full, 1); mbar_init(sdp_empty, 16); mbar_init(pds_full, 16); mbar_init(pds_empty, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmDO);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, BWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tAcc = tmem_base + 256;     // ACCBUF accumulator sets of 2 * HSP columns

    // one 128-row tile = NC boxes of 64 channels
    auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int slot, int row0, int b) {
        #pragma unroll
        for (int c = 0; c < NC; c++) tma_load_4d(dst + c * CHUNK_BYTES, tm, bar, c * 64, slot, row0, b);
    };

    if (warp == 0) {
        if (lane == 0) {
            int xst = 0; uint32_t xph = 0;                    // stream ring position of the next tile to load
            int it = 0;
            for (int w = blockIdx.x; w < total; w += gridDim.x, it++) {
                int fixed, b, h, cnt; decode(w, fixed, b, h, cnt);
                const int rb = it % RB;
                if (!mbar_wait(&res_empty[rb], ((it / RB) & 1) ^ 1, abort_flag, a.status, 0x601)) break;
                uint8_t* rdst = sRes + rb * PAIR_BYTES;
                mbar_expect_tx(&res_full[rb], PAIR_BYTES);
                if (DKV) {
                    load_tile(rdst, &tmQKV, &res_full[rb], a.NH + h, fixed * BT, b);                   // K_j
                    load_tile(rdst + TILE_BYTES, &tmQKV, &res_full[rb], 2 * a.NH + h, fixed * BT, b);  // V_j
                } else {
                    load_tile(rdst, &tmQKV, &res_full[rb], h, fixed * BT, b);                          // Q_i
                    load_tile(rdst + TILE_BYTES, &tmDO, &res_full[rb], h, fixed * BT, b);              // dO_i
                }
                bool fail = false;
                for (int n = 0; n < cnt; n++) {
                    const int st = xst;
                    if (!mbar_wait(&x_empty[st], xph ^ 1, abort_flag, a.status, 0x600)) { fail = true; break; }
                    if (++xst == XSTAGES) { xst = 0; xph ^= 1; }
                    uint8_t* dst = sStr + st * PAIR_BYTES;
                    mbar_expect_tx(&x_full[st], PAIR_BYTES);
                    if (DKV) {
                        const int i = fixed + n;
                        load_tile(dst, &tmQKV, &x_full[st], h, i * BT, b);                        // Q_i
                        load_tile(dst + TILE_BYTES, &tmDO, &x_full[st], h, i * BT, b);            // dO_i
                    } else {
                        load_tile(dst, &tmQKV, &x_full[st], a.NH + h, n * BT, b);                 // K_j
                        load_tile(dst + TILE_BYTES, &tmQKV, &x_full[st], 2 * a.NH + h, n * BT, b);// V_j
                    }
                }
                if (fail) break;
            }
        }
    } else if (warp == 1) {
        // ---- issuer of the score products S = Q K^T and dP = dO V^T.  Tile g + 1 is issued as soon as the softmax threads hold
        //      tile g in registers, so it runs underneath their exponentials.
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BT, 0, 0);
            uint32_t t = 0;
            int st = 0; uint32_t ph = 0;                      // stream ring position of tile t
            int it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x, it++) {
                int fixed, b, h, cnt; decode(w, fixed, b, h, cnt);
                const int rb = it % RB;
                ok = mbar_wait(&res_full[rb], (it / RB) & 1, abort_flag, a.status, 0x610);
                for (int n = 0; n < cnt && ok; n++, t++) {
                    ok = ok && mbar_wait(&x_full[st], ph, abort_flag, a.status, 0x612);
                    if (t > 0) ok = ok && mbar_wait(sdp_empty, (t - 1) & 1, abort_flag, a.status, 0x613);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t xs = smem_u32(sStr + st * PAIR_BYTES), rs = smem_u32(sRes + rb * PAIR_BYTES);
                    const uint32_t q = DKV ? xs : rs, dO = (DKV ? xs : rs) + TILE_BYTES;
                    const uint32_t k = DKV ? rs : xs, v = (DKV ? rs : xs) + TILE_BYTES;
                    #pragma unroll
                    for (int kk = 0; kk < HSP / 16; kk++) {      // 64-channel chunks are 16 KB apart, 16 channels = 32 bytes inside a chunk
                        const uint32_t off = (kk >> 2) * CHUNK_BYTES + (kk & 3) * 32;
                        umma_ss(tS, umma_desc_sw128(q + off, 16, 1024), umma_desc_sw128(k + off, 16, 1024), idesc_s, kk > 0);
                    }
                    #pragma unroll
                    for (int kk = 0; kk < HSP / 16; kk++) {
                        const uint32_t off = (kk >> 2) * CHUNK_BYTES + (kk & 3) * 32;
                        umma_ss(tdP, umma_desc_sw128(dO + off, 16, 1024), umma_desc_sw128(v + off, 16, 1024), idesc_s, kk > 0);
                    }
                    umma_commit(sdp_full);
                    if (n == cnt - 1) umma_commit(&res_empty[rb]);     // the resident pair is only read by these two products
                    if (++st == XSTAGES) { st = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == BWD_THREADS / 32 - 1) {
        // ---- issuer of the accumulating products (dV += P^T dO, dK += dS^T Q, or dQ += dS K).  A second issuing thread: a
        //      tcgen05.mma costs its issuer about a hundred cycles whatever its shape, and the two streams of products depend on
        //      different events, so two threads keep the tensor pipe fed where one could not.
        if (lane == 0) {
            constexpr uint32_t idesc_acc = DKV ? umma_idesc_bf16(BT, HSP, 1, 1) : umma_idesc_bf16(BT, HSP, 0, 1);
            uint32_t t = 0;
            int cst = 0;
            int it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x, it++) {
                int fixed, b, h, cnt; decode(w, fixed, b, h, cnt);
                const int ab = it % ACCBUF;
                const uint32_t acc0 = tAcc + ab * (2 * HSP), acc1 = acc0 + HSP;
                ok = mbar_wait(&acc_empty[ab], ((it / ACCBUF) & 1) ^ 1, abort_flag, a.status, 0x616);
                for (int n = 0; n < cnt && ok; n++, t++) {
                    ok = mbar_wait(pds_full, t & 1, abort_flag, a.status, 0x614);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t xs = smem_u32(sStr + cst * PAIR_BYTES);
                    const uint32_t p = smem_u32(sP), ds = smem_u32(sdS);
                    if (DKV) {
                        // dV += P^T dO ; dK += dS^T Q : A is MN-major (two 64-wide groups 16 KB apart), K = 128 query rows;
                        // B = dO / Q tile as an N-major operand (NC groups of 64 channels, 16 KB apart)
                        #pragma unroll
                        for (int kk = 0; kk < BT / 16; kk++)
                            umma_ss(acc0, umma_desc_sw128(p + kk * 2048, BT * 128, 1024), umma_desc_sw128(xs + TILE_BYTES + kk * 2048, CHUNK_BYTES, 1024),
                                    idesc_acc, (n > 0 || kk > 0));
                        #pragma unroll
                        for (int kk = 0; kk < BT / 16; kk++)
                            umma_ss(acc1, umma_desc_sw128(ds + kk * 2048, BT * 128, 1024), umma_desc_sw128(xs + kk * 2048, CHUNK_BYTES, 1024),
                                    idesc_acc, (n > 0 || kk > 0));
                    } else {
                        // dQ += dS K : A K-major (two 64-column chunks), B = K_j as an N-major operand
                        #pragma unroll
                        for (int kk = 0; kk < BT / 16; kk++)
                            umma_ss(acc0, umma_desc_sw128(ds + (kk >> 2) * (BT * 128) + (kk & 3) * 32, 16, 1024),
                                    umma_desc_sw128(xs + kk * 2048, CHUNK_BYTES, 1024), idesc_acc, (n > 0 || kk > 0));
                    }
                    umma_commit(&x_empty[cst]);
                    umma_commit(pds_empty);
                    if (n == cnt - 1) umma_commit(&acc_full[ab]);
                    if (++cst == XSTAGES) cst = 0;
                }
            }
        }
    } else {
        // softmax / epilogue: thread = one row x one 32-column quarter of the 128 x 128 tile.
        // These warps never leave their loops early: after an abandoned wait every later wait returns at once.
        const int q = warp & 3;                        // TMEM lane quarter
        const int cq = (warp - 2) >> 2;                // column quarter handled by this thread
        const int r = q * 32 + lane;                   // row of the tile (a query row in S / dP)
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const float log2e = 1.4426950408889634f;
        bool ok = true;
        uint32_t t = 0;
        int it = 0;
        for (int w = blockIdx.x; w < total; w += gridDim.x, it++) {
            int fixed, b, h, cnt; decode(w, fixed, b, h, cnt);
            const size_t stat_base = ((size_t)b * a.NH + h) * a.T;
            float lse_l2 = 0.f, dlt_s = 0.f;           // LSE in log2 units; delta pre-multiplied by the softmax scale
            bool row_ok;
            {
                const int t0 = fixed * BT + r;
                row_ok = t0 < a.T;
                if (row_ok) { lse_l2 = a.lse[stat_base + t0] * log2e; dlt_s = a.delta[stat_base + t0] * a.scale; }
            }
            for (int n = 0; n < cnt; n++, t++) {
                const int qi = DKV ? fixed + n : fixed;    // query tile index
                const int kj = DKV ? fixed : n;            // key tile index
                // prefetch the next query tile's statistics (only the dK/dV kernel changes rows between tiles)
                float nxt_lse = 0.f, nxt_dlt = 0.f; bool nxt_ok = row_ok;
                const bool fetch_next = DKV && n + 1 < cnt;
                if (fetch_next) {
                    const int tn = (qi + 1) * BT + r;
                    nxt_ok = tn < a.T;
                    if (nxt_ok) { nxt_lse = a.lse[stat_base + tn]; nxt_dlt = a.delta[stat_base + tn]; } else { nxt_lse = 0.f; nxt_dlt = 0.f; }     // raw: converted below, after the loads had a whole tile to land
                }
                ok = mbar_wait(sdp_full, t & 1, abort_flag, a.status, 0x620) && ok;
                tc_fence_after();
                uint32_t sv[32], dv[32];
                tmem_ld32(tS + lane_off + cq * 32, sv);
                tmem_ld32(tdP + lane_off + cq * 32, dv);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sdp_empty);      // S / dP may be overwritten by the next tile
                uint32_t pp[16], dd[16];
                if (qi == kj || !row_ok) {
                    // diagonal tile (or rows past the end of the sequence): mask above the diagonal
                    #pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int c0 = cq * 32 + e;
                        float p0 = ex2_fast(fmaf(__uint_as_float(sv[e]), a.scale_log2e, -lse_l2));
                        float p1 = ex2_fast(fmaf(__uint_as_float(sv[e + 1]), a.scale_log2e, -lse_l2));
                        if (!row_ok || c0 > r) p0 = 0.f;
                        if (!row_ok || c0 + 1 > r) p1 = 0.f;
                        const float d0 = p0 * fmaf(__uint_as_float(dv[e]), a.scale, -dlt_s);
                        const float d1 = p1 * fmaf(__uint_as_float(dv[e + 1]), a.scale, -dlt_s);
                        pp[e >> 1] = pack_bf16x2(p0, p1);
                        dd[e >> 1] = pack_bf16x2(d0, d1);
                    }
                } else {
                    #pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float p0 = ex2_fast(fmaf(__uint_as_float(sv[e]), a.scale_log2e, -lse_l2));
                        const float p1 = ex2_fast(fmaf(__uint_as_float(sv[e + 1]), a.scale_log2e, -lse_l2));
                        const float d0 = p0 * fmaf(__uint_as_float(dv[e]), a.scale, -dlt_s);
                        const float d1 = p1 * fmaf(__uint_as_float(dv[e + 1]), a.scale, -dlt_s);
                        pp[e >> 1] = pack_bf16x2(p0, p1);
                        dd[e >> 1] = pack_bf16x2(d0, d1);
                    }
                }
                if (t > 0) ok = mbar_wait(pds_empty, (t - 1) & 1, abort_flag, a.status, 0x621) && ok;   // previous tile's MMAs have read P / dS
                // 64-column chunk (cq >> 1), 16-byte units (cq & 1) * 4 .. +3 of this row, 128-byte swizzle
                uint8_t* prow = sP + (cq >> 1) * (BT * 128) + r * 128;
                uint8_t* drow = sdS + (cq >> 1) * (BT * 128) + r * 128;
                #pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int pos = ((((cq & 1) * 4) + u) ^ (r & 7)) * 16;
                    if (DKV) *reinterpret_cast<uint4*>(prow + pos) = make_uint4(pp[u * 4], pp[u * 4 + 1], pp[u * 4 + 2], pp[u * 4 + 3]);
                    *reinterpret_cast<uint4*>(drow + pos) = make_uint4(dd[u * 4], dd[u * 4 + 1], dd[u * 4 + 2], dd[u * 4 + 3]);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(pds_full);
                if (fetch_next) { lse_l2 = nxt_lse * log2e; dlt_s = nxt_dlt * a.scale; row_ok = nxt_ok; }
            }
            // ---- item epilogue: accumulators -> global; the issuing warps are already working on the next item
            const int ab = it % ACCBUF;
            ok = mbar_wait(&acc_full[ab], (it / ACCBUF) & 1, abort_flag, a.status, 0x622) && ok;
            tc_fence_after();
            uint32_t v0[16 * NC], v1[16 * NC];
            #pragma unroll
            for (int c = 0; c < NC; c++) {
                tmem_ld16(tAcc + ab * (2 * HSP) + c * 64 + lane_off + cq * 16, v0 + c * 16);
                if (DKV) tmem_ld16(tAcc + ab * (2 * HSP) + HSP + c * 64 + lane_off + cq * 16, v1 + c * 16);
            }
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
            const int trow = fixed * BT + r;
            if (trow < a.T && ok) {
                // DKV: acc0 = dV (slot 2), acc1 = dK (slot 1); else acc0 = dQ (slot 0)
                bf16* dst0 = a.dqkv + (((size_t)b * a.T + trow) * 3 + (DKV ? 2 : 0)) * a.NH * a.hs + (size_t)h * a.hs;
                bf16* dst1 = a.dqkv + (((size_t)b * a.T + trow) * 3 + 1) * a.NH * a.hs + (size_t)h * a.hs;
                #pragma unroll
                for (int c = 0; c < NC; c++) {
                    #pragma unroll
                    for (int e = 0; e < 16; e += 8) {
                        const int col = c * 64 + cq * 16 + e;
                        if (col < a.hs) {
                            const uint32_t* x0 = v0 + c * 16 + e;
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(x0[0]), __uint_as_float(x0[1])); o.y = pack_bf16x2(__uint_as_float(x0[2]), __uint_as_float(x0[3]));
                            o.z = pack_bf16x2(__uint_as_float(x0[4]), __uint_as_float(x0[5])); o.w = pack_bf16x2(__uint_as_float(x0[6]), __uint_as_float(x0[7]));
                            *reinterpret_cast<uint4*>(dst0 + col) = o;
                            if (DKV) {
                                const uint32_t* x1 = v1 + c * 16 + e;
                                o.x = pack_bf16x2(__uint_as_float(x1[0]), __uint_as_float(x1[1])); o.y = pack_bf16x2(__uint_as_float(x1[2]), __uint_as_float(x1[3]));
                                o.z = pack_bf16x2(__uint_as_float(x1[4]), __uint_as_float(x1[5])); o.w = pack_bf16x2(__uint_as_float(x1[6]), __uint_as_float(x1[7]));
                                *reinterpret_cast<uint4*>(dst1 + col) = o;
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {
        long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, BWD_TMEM_COLS);
}

}  // namespace

template <int NC>
int launch_bwd(const CUtensorMap& tmQKV, const CUtensorMap& tmDO, const BwdArgs& a, int grid, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<true, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<NC>::SMEM));
        CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<false, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<NC>::SMEM));
        configured = true;
    }
    attn_bwd_kernel<true, NC><<<grid, BWD_THREADS, BwdCfg<NC>::SMEM, stream>>>(tmQKV, tmDO, a);
    CUDA_CHECK(cudaGetLastError());
    attn_bwd_kernel<false, NC><<<grid, BWD_THREADS, BwdCfg<NC>::SMEM, stream>>>(tmQKV, tmDO, a);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// delta[b,h,t] = sum_d O[b,t,h,d] * dO[b,t,h,d] (shared with the single-pass kernel of attention_bwd1.cu)
int llmc_attention_delta(float* delta, const bf16* out, const bf16* dout, int B, int T, int NH, int hs, cudaStream_t stream) {
    const long long rows = (long long)B * T * NH;
    delta_kernel<<<(unsigned)CEIL_DIV(rows * 8, 256), 256, 0, stream>>>(delta, out, dout, B, T, NH, hs);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// dqkv (B,T,3,NH,HS) = gradient of causal attention; delta: scratch of B*NH*T floats.  Head sizes: multiples of 8, 64..128.
// The entry point llmc_attention_bwd (attention_bwd1.cu) sends every head size but 64 here.
int llmc_attention_bwd_two_pass(bf16* dqkv, float* delta, const bf16* dout, const bf16* qkv, const bf16* out, const float* lse,
                                int B, int T, int NH, int hs, cudaStream_t stream) {
    if (hs < 64 || hs > 128 || (hs % 8)) { fprintf(stderr, "[llmc_b200] attention backward: head size %d not supported (multiples of 8 from 64 to 128)\n", hs); return -1; }
    CUtensorMap tmQKV, tmDO;
    int rc = llmc_attn_qkv_map(&tmQKV, qkv, B, T, NH, hs);
    if (rc) return rc;
    {
        uint64_t dims[4] = {(uint64_t)hs, (uint64_t)NH, (uint64_t)T, (uint64_t)B};
        uint64_t strides[4] = {2, (uint64_t)hs * 2, (uint64_t)NH * hs * 2, (uint64_t)T * NH * hs * 2};
        uint32_t box[4] = {64, 1, 128, 1};
        if ((rc = llmc_get_tensormap(&tmDO, dout, 2, 4, dims, strides, box, 3))) return rc;
    }
    if ((rc = llmc_attention_delta(delta, out, dout, B, T, NH, hs, stream))) return rc;
    BwdArgs a;
    a.dqkv = dqkv; a.lse = lse; a.delta = delta; a.B = B; a.T = T; a.NH = NH; a.hs = hs;
    a.scale = 1.0f / sqrtf((float)hs);
    a.scale_log2e = a.scale * 1.4426950408889634f;
    a.status = llmc_status_ptr();
    const int nt = CEIL_DIV(T, BT);
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int grid = B * NH * nt < sms ? B * NH * nt : sms;
    return hs <= 64 ? launch_bwd<1>(tmQKV, tmDO, a, grid, stream) : launch_bwd<2>(tmQKV, tmDO, a, grid, stream);
}
