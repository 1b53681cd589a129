// Causal flash attention forward for sm_100a on the packed (B, T, 3, NH, HS) QKV layout; head sizes 64..128
// (multiples of 8; sizes above 64 run as a 128-wide head whose missing channels TMA fills with zeros).
//
// Persistent: one CTA per SM walks a heavy-first list of (batch, head, 128-row query tile) work items; Q is double
// buffered so the next item's loads and first MMA run under the current item's tail.  Roles inside a CTA (576 threads):
//   warp 0      TMA producer: Q once, then K and V tiles (double buffered), read in place from the
//               packed QKV tensor through a 4-D tensor map.
//   warp 1      MMA issuer: S = Q K^T into TMEM columns [0,128), PV = P V into one of two 64-column
//               TMEM buffers.  S(j+1) is issued as soon as the softmax threads hold S(j) in registers.
//   warps 2-17  softmax: thread = query row x 32-column quarter.  One TMEM load of its 32 scores, row
//               maximum exchanged between the four quarters through shared memory, exp2 on the SFU,
//               bf16 P written to 128-byte-swizzled shared memory (A operand of the PV MMA, double
//               buffered); each thread owns 16 of the 64 output columns in registers and folds in the
//               previous tile's PV while the tensor core works on the current one.
// Statistics are written as natural-log LSE per (b, h, t), the layout cuDNN's SDPA uses in the
// reference (llmc/cudnn_att.cpp:105-113).  Tiles above the diagonal are skipped.
//
// Capability parity: attention_forward_cudnn (llmc/cudnn_att.cpp:222-254) and the unfused
// attention_forward of llmc/attention.cuh in the reference.
#include "common.cuh"

namespace {

constexpr int BQ = 128, BKV = 128;
constexpr int CHUNK_BYTES = 128 * 64 * 2;          // 16 KB: 128 rows x 64 channels of bf16, one 128-byte-swizzled TMA box
constexpr int P_BYTES = BQ * BKV * 2;              // 32 KB
constexpr int XCH_BYTES = (2 * 4 * 128 + 4 * 128) * 4;     // row-max exchange (double buffered) + final row sums
constexpr int FWD_THREADS = 576;                   // TMA warp + MMA warp + 16 softmax warps

// NC = number of 64-channel chunks of the (zero-padded) head: 1 -> head size 64, 2 -> head sizes 72..128.
// The wider variant trades buffering for capacity (single Q / P buffers, two K/V stages) to stay within shared memory.
template <int NC> struct FwdCfg {
    static constexpr int HSP = 64 * NC;
    static constexpr int TILE_BYTES = NC * CHUNK_BYTES;
    static constexpr int QBUF = NC == 1 ? 2 : 1;
    static constexpr int KVSTAGES = NC == 1 ? 3 : 2;
    static constexpr int PBUF = NC == 1 ? 2 : 1;
    static constexpr int SMEM = QBUF * TILE_BYTES + 2 * KVSTAGES * TILE_BYTES + PBUF * P_BYTES + XCH_BYTES + 256;
    static constexpr int TMEM_COLS = NC == 1 ? 256 : 512;      // S (128) + two O buffers of HSP columns
};

struct FwdArgs {
    bf16* out;         // (B, T, NH, HS)
    float* lse;        // (B, NH, T)
    int B, T, NH, hs;
    float scale_log2e; // (1/sqrt(HS)) * log2(e)
    float scale;
    unsigned int* status;
};

DEVINL void quarter_barrier(int q) { asm volatile("bar.sync %0, 128;" ::"r"(1 + q) : "memory"); }

template <int NC>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const FwdArgs a) {
    using Cfg = FwdCfg<NC>;
    constexpr int HSP = Cfg::HSP, TILE_BYTES = Cfg::TILE_BYTES, QBUF = Cfg::QBUF, KVSTAGES = Cfg::KVSTAGES, PBUF = Cfg::PBUF;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                        // QBUF buffers (current / next work item)
    uint8_t* sK = sQ + QBUF * TILE_BYTES;      // KVSTAGES stages
    uint8_t* sV = sK + KVSTAGES * TILE_BYTES;  // KVSTAGES stages
    uint8_t* sP = sV + KVSTAGES * TILE_BYTES;  // PBUF buffers
    float* xmax = reinterpret_cast<float*>(sP + PBUF * P_BYTES);   // [2][4][128]
    float* xsum = xmax + 2 * 4 * 128;                              // [4][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xmax) + XCH_BYTES);
    uint64_t* q_full = bars + 0;     // [2]
    uint64_t* q_empty = bars + 2;    // [2]
    uint64_t* k_full = bars + 4;     // [KVSTAGES]
    uint64_t* k_empty = bars + 8;    // [KVSTAGES]
    uint64_t* v_full = bars + 12;    // [KVSTAGES]
    uint64_t* v_empty = bars + 16;   // [KVSTAGES]
    uint64_t* s_full = bars + 20;
    uint64_t* s_empty = bars + 21;
    uint64_t* p_full = bars + 22;
    uint64_t* o_full = bars + 23;    // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nq = CEIL_DIV(a.T, BQ);
    const int BH = a.B * a.NH;
    const int total = BH * nq;
    // persistent: work item w -> (query tile, batch, head); late (heavy) query tiles first
    auto decode = [&](int w, int& qi, int& b, int& h) {
        const int rank = w / BH, bh = w - rank * BH;
        qi = nq - 1 - rank;
        b = bh / a.NH; h = bh - b * a.NH;
    };

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) record_error(a.status, ST_BAD_ARG, 0x10);
        for (int i = 0; i < 2; i++) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); mbar_init(&o_full[i], 1); }
        for (int i = 0; i < KVSTAGES; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
        mbar_init(s_full, 1); mbar_init(s_empty, 16); mbar_init(p_full, 16);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tO = tmem_base + 128;       // O partial products: two buffers of HSP columns

    if (warp == 0) {
        if (lane == 0) {
            int kst = 0; uint32_t kph = 0;
            int it = 0;
            for (int w = blockIdx.x; w < total; w += gridDim.x, it++) {
                int qi, b, h; decode(w, qi, b, h);
                const int qb = it % QBUF;
                if (!mbar_wait(&q_empty[qb], ((it / QBUF) & 1) ^ 1, abort_flag, a.status, 0x502)) break;
                mbar_expect_tx(&q_full[qb], TILE_BYTES);
                #pragma unroll
                for (int c = 0; c < NC; c++) tma_load_4d(sQ + qb * TILE_BYTES + c * CHUNK_BYTES, &tmQKV, &q_full[qb], c * 64, h, qi * BQ, b);
                bool fail = false;
                for (int j = 0; j <= qi; j++) {
                    const int st = kst;
                    const uint32_t ph = kph ^ 1;
                    if (++kst == KVSTAGES) { kst = 0; kph ^= 1; }
                    if (!mbar_wait(&k_empty[st], ph, abort_flag, a.status, 0x500)) { fail = true; break; }
                    mbar_expect_tx(&k_full[st], TILE_BYTES);
                    #pragma unroll
                    for (int c = 0; c < NC; c++) tma_load_4d(sK + st * TILE_BYTES + c * CHUNK_BYTES, &tmQKV, &k_full[st], c * 64, a.NH + h, j * BKV, b);
                    if (!mbar_wait(&v_empty[st], ph, abort_flag, a.status, 0x501)) { fail = true; break; }
                    mbar_expect_tx(&v_full[st], TILE_BYTES);
                    #pragma unroll
                    for (int c = 0; c < NC; c++) tma_load_4d(sV + st * TILE_BYTES + c * CHUNK_BYTES, &tmQKV, &v_full[st], c * 64, 2 * a.NH + h, j * BKV, b);
                }
                if (fail) break;
            }
        }
    } else if (warp == 1) {
        // The whole warp runs the issuing code in uniform control flow and one elected lane executes the tcgen05 instructions: a
        // single lane inside a divergent branch has to move every descriptor from its registers to uniform registers, which costs
        // it about 90 cycles per product (measured), more than a 128 x 64 x 16 product runs.  Wait results go through a warp vote
        // so that the compiler knows the branches on them to be uniform; descriptors are built once and advanced by addition.
        {
            const bool leader = elect_one();
#define WAIT_ALL(bar, parity, code) (__all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, a.status, code)) != 0)
            constexpr uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, 0, 0);     // Q (K-major) x K (K-major)
            constexpr uint32_t idesc_o = umma_idesc_bf16(BQ, HSP, 0, 1);     // P (K-major) x V (N-major)
            constexpr uint32_t TILE_UNITS = TILE_BYTES / 16, P_UNITS = P_BYTES / 16;
            const uint64_t dQ0 = umma_desc_sw128(smem_u32(sQ), 16, 1024), dK0 = umma_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t dP0 = umma_desc_sw128(smem_u32(sP), 16, 1024), dV0 = umma_desc_sw128(smem_u32(sV), CHUNK_BYTES, 1024);
            auto issue_s = [&](int st, int qb, bool last_of_item) {
                const uint64_t q = dQ0 + (uint32_t)qb * TILE_UNITS, k = dK0 + (uint32_t)st * TILE_UNITS;
                if (leader) {
                    #pragma unroll
                    for (int kk = 0; kk < HSP / 16; kk++) {      // 64-channel chunks are 16 KB apart, 16 channels = 32 bytes inside a chunk
                        const uint32_t off = ((kk >> 2) * CHUNK_BYTES + (kk & 3) * 32) / 16;
                        umma_ss(tS, q + off, k + off, idesc_s, kk > 0);
                    }
                    umma_commit(s_full);
                    umma_commit(&k_empty[st]);
                    if (last_of_item) umma_commit(&q_empty[qb]);
                }
            };
            uint32_t t = 0;
            int cst = 0; uint32_t cph = 0;        // K/V ring position of tile t
            int it = 0;
            bool ok = true;
            if ((int)blockIdx.x < total) {
                int qi, b, h; decode(blockIdx.x, qi, b, h);
                ok = WAIT_ALL(&q_full[0], 0, 0x510) && WAIT_ALL(&k_full[0], 0, 0x511);
                tc_fence_after();
                if (ok) issue_s(0, 0, qi == 0);
            }
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x, it++) {
                int qi, b, h; decode(w, qi, b, h);
                for (int j = 0; j <= qi && ok; j++, t++) {
                    // S of the next tile (possibly the first tile of the next work item) as soon as S(t) sits in registers
                    bool have_next = true, new_item = false; int nqi = qi, nj = j + 1;
                    if (nj > qi) {
                        if (w + (int)gridDim.x < total) { int b2, h2; decode(w + gridDim.x, nqi, b2, h2); nj = 0; new_item = true; }
                        else have_next = false;
                    }
                    if (have_next) {
                        const int nit = it + (new_item ? 1 : 0);
                        if (new_item) ok = ok && WAIT_ALL(&q_full[nit % QBUF], (nit / QBUF) & 1, 0x516);
                        int nst = cst + 1; uint32_t nph = cph;
                        if (nst == KVSTAGES) { nst = 0; nph ^= 1; }
                        ok = ok && WAIT_ALL(&k_full[nst], nph, 0x512);
                        ok = ok && WAIT_ALL(s_empty, t & 1, 0x513);
                        if (!ok) break;
                        tc_fence_after();
                        issue_s(nst, nit % QBUF, nj == nqi);
                    }
                    ok = ok && WAIT_ALL(p_full, t & 1, 0x514);
                    ok = ok && WAIT_ALL(&v_full[cst], cph, 0x515);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t p = dP0 + (uint32_t)(t % PBUF) * P_UNITS, v = dV0 + (uint32_t)cst * TILE_UNITS;
                    if (leader) {
                        #pragma unroll
                        for (int kk = 0; kk < BKV / 16; kk++) {
                            // P: two 64-column swizzled chunks of 16 KB; V: 128 kv rows of 128 B, 16 rows per K step
                            umma_ss(tO + (t & 1) * HSP, p + ((kk >> 2) * (BQ * 128) + (kk & 3) * 32) / 16, v + kk * 128, idesc_o, kk > 0);
                        }
                        umma_commit(&o_full[t & 1]);
                        umma_commit(&v_empty[cst]);
                    }
                    if (++cst == KVSTAGES) { cst = 0; cph ^= 1; }
                }
            }
#undef WAIT_ALL
        }
    } else {
        // softmax: thread = query row r x 32-column quarter cq of the S tile; it also owns 16 of the 64 output columns.
        // These warps meet at named barriers, so they never leave the loops early (abandoned waits return at once).
        const int q = warp & 3;
        const int cq = (warp - 2) >> 2;
        const int r = q * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        bool ok = true;
        uint32_t t = 0;
        for (int w = blockIdx.x; w < total; w += gridDim.x) {
            int qi, b, h; decode(w, qi, b, h);
            float m = -INFINITY, l = 0.f;
            float O[16 * NC];                  // columns c*64 + cq*16 .. +15 of every 64-channel chunk c
            #pragma unroll
            for (int d = 0; d < 16 * NC; d++) O[d] = 0.f;
            // adds the finished P V of tile `tt` to the running output (optionally rescaled afterwards)
            auto fold = [&](uint32_t tt, float rescale) {
                ok = mbar_wait(&o_full[tt & 1], (tt >> 1) & 1, abort_flag, a.status, 0x521) && ok;
                tc_fence_after();
                #pragma unroll
                for (int c = 0; c < NC; c++) {
                    uint32_t ov[16];
                    tmem_ld16(tO + (tt & 1) * HSP + c * 64 + lane_off + cq * 16, ov);
                    tmem_ld_wait();
                    #pragma unroll
                    for (int d = 0; d < 16; d++) O[c * 16 + d] = (O[c * 16 + d] + __uint_as_float(ov[d])) * rescale;
                }
                tc_fence_before();
            };
            for (int j = 0; j <= qi; j++, t++) {
                ok = mbar_wait(s_full, t & 1, abort_flag, a.status, 0x520) && ok;
                tc_fence_after();
                uint32_t v[32];
                tmem_ld32(tS + lane_off + cq * 32, v);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty);
                float mx = -INFINITY;
                if (j == qi) {
                    #pragma unroll
                    for (int e = 0; e < 32; e++) {
                        if (cq * 32 + e > r) v[e] = 0xff800000u;      // -inf: above the diagonal
                        mx = fmaxf(mx, __uint_as_float(v[e]));
                    }
                } else {
                    #pragma unroll
                    for (int e = 0; e < 32; e++) mx = fmaxf(mx, __uint_as_float(v[e]));
                }
                // row maximum over the four column quarters
                float* xm = xmax + (t & 1) * 512;
                xm[cq * 128 + r] = mx;
                quarter_barrier(q);
                mx = fmaxf(fmaxf(xm[r], xm[128 + r]), fmaxf(xm[256 + r], xm[384 + r]));
                const float m_new = fmaxf(m, mx);
                const float alpha = ex2_fast((m - m_new) * a.scale_log2e);      // m = -inf on the first tile -> 0
                m = m_new;
                const float moff = m * a.scale_log2e;
                float rs = 0.f;
                uint32_t pk[16];
                #pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = ex2_fast(fmaf(__uint_as_float(v[e]), a.scale_log2e, -moff));
                    const float p1 = ex2_fast(fmaf(__uint_as_float(v[e + 1]), a.scale_log2e, -moff));
                    rs += p0 + p1;
                    pk[e >> 1] = pack_bf16x2(p0, p1);
                }
                l = l * alpha + rs;
                if (PBUF == 1 && j > 0) fold(t - 1, alpha);      // single P buffer: the previous P V must have consumed it
                uint8_t* prow = sP + (t % PBUF) * P_BYTES + (cq >> 1) * (BQ * 128) + r * 128;
                #pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int pos = ((((cq & 1) * 4) + u) ^ (r & 7)) * 16;
                    *reinterpret_cast<uint4*>(prow + pos) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                // fold in the previous tile's P V (rescaled to the new maximum together with the running output)
                if (PBUF != 1 && j > 0) fold(t - 1, alpha);
            }
            fold(t - 1, 1.0f);      // last tile of the item
            // total row sum over the four quarters
            xsum[cq * 128 + r] = l;
            quarter_barrier(q);
            l = xsum[r] + xsum[128 + r] + xsum[256 + r] + xsum[384 + r];
            const int trow = qi * BQ + r;
            if (trow < a.T && ok) {
                const float inv = 1.0f / l;
                bf16* op = a.out + (((size_t)b * a.T + trow) * a.NH + h) * a.hs;
                #pragma unroll
                for (int c = 0; c < NC; c++) {
                    #pragma unroll
                    for (int d = 0; d < 16; d += 8) {
                        const int col = c * 64 + cq * 16 + d;
                        if (col < a.hs) {          // head sizes are multiples of 8: whole 16-byte groups
                            const float* Oc = O + c * 16 + d;
                            uint4 o;
                            o.x = pack_bf16x2(Oc[0] * inv, Oc[1] * inv); o.y = pack_bf16x2(Oc[2] * inv, Oc[3] * inv);
                            o.z = pack_bf16x2(Oc[4] * inv, Oc[5] * inv); o.w = pack_bf16x2(Oc[6] * inv, Oc[7] * inv);
                            *reinterpret_cast<uint4*>(op + col) = o;
                        }
                    }
                }
                if (cq == 0) a.lse[((size_t)b * a.NH + h) * a.T + trow] = m * a.scale + logf(l);
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
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace

// Tensor map over a packed (B, T, 3, NH, HS) tensor seen as 4-D {HS, 3*NH, T, B} with a 128-row box.
int llmc_attn_qkv_map(CUtensorMap* tm, const bf16* qkv, int B, int T, int NH, int hs) {
    uint64_t dims[4] = {(uint64_t)hs, (uint64_t)(3 * NH), (uint64_t)T, (uint64_t)B};
    uint64_t strides[4] = {2, (uint64_t)hs * 2, (uint64_t)3 * NH * hs * 2, (uint64_t)T * 3 * NH * hs * 2};
    uint32_t box[4] = {64, 1, 128, 1};
    return llmc_get_tensormap(tm, qkv, 2, 4, dims, strides, box, 3);
}

template <int NC>
int launch_fwd(const CUtensorMap& tm, const FwdArgs& a, int grid, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<NC>::SMEM));
        configured = true;
    }
    attn_fwd_kernel<NC><<<grid, FWD_THREADS, FwdCfg<NC>::SMEM, stream>>>(tm, a);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// out (B,T,NH,HS) = causal softmax(Q K^T / sqrt(HS)) V ; lse (B,NH,T) fp32.  Head sizes: multiples of 8 up to 128.
// The entry point llmc_attention_fwd (attention_fwd1.cu) sends every head size but 64 here.
int llmc_attention_fwd_general(bf16* out, float* lse, const bf16* qkv, int B, int T, int NH, int hs, cudaStream_t stream) {
    if (hs < 64 || hs > 128 || (hs % 8)) { fprintf(stderr, "[llmc_b200] attention: head size %d not supported (multiples of 8 from 64 to 128)\n", hs); return -1; }
    CUtensorMap tm;
    int rc = llmc_attn_qkv_map(&tm, qkv, B, T, NH, hs);
    if (rc) return rc;
    FwdArgs a;
    a.out = out; a.lse = lse; a.B = B; a.T = T; a.NH = NH; a.hs = hs;
    a.scale = 1.0f / sqrtf((float)hs);
    a.scale_log2e = a.scale * 1.4426950408889634f;
    a.status = llmc_status_ptr();
    const int nq = CEIL_DIV(T, BQ);
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int grid = B * NH * nq < sms ? B * NH * nq : sms;
    return hs <= 64 ? launch_fwd<1>(tm, a, grid, stream) : launch_fwd<2>(tm, a, grid, stream);
}
