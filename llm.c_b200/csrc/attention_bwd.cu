// Causal flash attention backward for sm_100a on the packed (B, T, 3, NH, HS) layout, HS = 64.
//
// Deterministic by construction: no atomics, every output element has one writer and a fixed
// summation order.  Three launches:
//   1. delta[b,h,t] = sum_d O[b,t,h,d] * dO[b,t,h,d]
//   2. "dK/dV" kernel: one CTA per (b, h, 128-row key/value tile).  K_j and V_j stay resident in
//      shared memory while the query tiles i >= j stream through a 2-stage TMA ring.  Per query tile
//      S = Q K^T and dP = dO V^T are formed in TMEM, the 256 softmax threads turn them into
//      P = exp(S*scale - LSE) and dS = P (dP - delta) scale (bf16, swizzled shared memory), and
//      dV += P^T dO, dK += dS^T Q accumulate in TMEM over the whole loop (MN-major A operands).
//   3. "dQ" kernel: one CTA per (b, h, query tile); K_j, V_j stream; dQ += dS K accumulates in TMEM.
// S and dP are recomputed in (3) instead of exchanging dQ partials through atomics; that costs two
// extra MMAs per tile and buys bit-reproducible gradients, which the reference also demands of
// cuDNN (llmc/cudnn_att.cpp:186-191).
//
// A CTA has 320 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 softmax/epilogue
// (thread = one row x one 64-column half).  The softmax threads pull S/dP into registers and release
// the TMEM tiles at once, so the next tile's S/dP MMAs run underneath the exponentials.
//
// Capability parity: attention_backward_cudnn (llmc/cudnn_att.cpp:256-288) and attention_backward
// of llmc/attention.cuh in the reference.
#include "common.cuh"

int llmc_attn_qkv_map(CUtensorMap* tm, const bf16* qkv, int B, int T, int NH, int hs);   // attention_fwd.cu

namespace {

constexpr int HS = 64;
constexpr int BT = 128;                             // tile rows (queries and keys)
constexpr int TILE_BYTES = BT * HS * 2;             // 16 KB
constexpr int PAIR_BYTES = 2 * TILE_BYTES;          // 32 KB
constexpr int PS_BYTES = BT * BT * 2;               // 32 KB
constexpr int BWD_SMEM = PAIR_BYTES /*resident*/ + 2 * PAIR_BYTES /*stream*/ + 2 * PS_BYTES /*P, dS*/ + 256;
constexpr int BWD_THREADS = 320;
constexpr int BWD_TMEM_COLS = 512;

struct BwdArgs {
    bf16* dqkv;          // (B, T, 3, NH, HS)
    const float* lse;    // (B, NH, T)
    const float* delta;  // (B, NH, T)
    int B, T, NH;
    float scale, scale_log2e;
    unsigned int* status;
};

__global__ void delta_kernel(float* __restrict__ delta, const bf16* __restrict__ out, const bf16* __restrict__ dout,
                             int B, int T, int NH) {
    // 8 lanes per (b, t, h) row of 64 channels
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = gid >> 3;
    const int part = (int)(gid & 7);
    const long long rows = (long long)B * T * NH;
    float acc = 0.f;
    if (row < rows) {
        bf16x8 o = ld128cs(out + row * HS + part * 8), d = ld128cs(dout + row * HS + part * 8);
        #pragma unroll
        for (int e = 0; e < 8; e++) acc += __bfloat162float(o[e]) * __bfloat162float(d[e]);
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
template <bool DKV>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO, const BwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sRes = smem;                              // [2][16 KB]
    uint8_t* sStr = sRes + PAIR_BYTES;                 // [2 stages][2][16 KB]
    uint8_t* sP = sStr + 2 * PAIR_BYTES;
    uint8_t* sdS = sP + PS_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + PS_BYTES);
    uint64_t* res_full = bars + 0;
    uint64_t* x_full = bars + 1;      // [2]
    uint64_t* x_empty = bars + 3;     // [2]
    uint64_t* sdp_full = bars + 5;
    uint64_t* sdp_empty = bars + 6;
    uint64_t* pds_full = bars + 7;
    uint64_t* pds_empty = bars + 8;
    uint64_t* acc_full = bars + 9;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = CEIL_DIV(a.T, BT);
    const int tile_rank = (int)(blockIdx.x / (a.B * a.NH));
    const int bh = blockIdx.x % (a.B * a.NH);
    const int b = bh / a.NH, h = bh % a.NH;
    // heavy tiles first: key tile 0 sees every query tile; query tile nt-1 sees every key tile
    const int fixed = DKV ? tile_rank : (nt - 1 - tile_rank);
    const int cnt = DKV ? (nt - fixed) : (fixed + 1);

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) record_error(a.status, ST_BAD_ARG, 0x20);
        mbar_init(res_full, 1);
        for (int i = 0; i < 2; i++) { mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1); }
        mbar_init(sdp_full, 1); mbar_init(sdp_empty, 8); mbar_init(pds_full, 8); mbar_init(pds_empty, 1); mbar_init(acc_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmDO);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, BWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tAcc0 = tmem_base + 256, tAcc1 = tmem_base + 320;

    if (warp == 0) {
        if (lane == 0) {
            // resident pair
            mbar_expect_tx(res_full, PAIR_BYTES);
            if (DKV) {
                tma_load_4d(sRes, &tmQKV, res_full, 0, a.NH + h, fixed * BT, b);                   // K_j
                tma_load_4d(sRes + TILE_BYTES, &tmQKV, res_full, 0, 2 * a.NH + h, fixed * BT, b);  // V_j
            } else {
                tma_load_4d(sRes, &tmQKV, res_full, 0, h, fixed * BT, b);                          // Q_i
                tma_load_4d(sRes + TILE_BYTES, &tmDO, res_full, 0, h, fixed * BT, b);              // dO_i
            }
            for (int n = 0; n < cnt; n++) {
                const int st = n & 1;
                if (!mbar_wait(&x_empty[st], ((n >> 1) & 1) ^ 1, abort_flag, a.status, 0x600)) break;
                uint8_t* dst = sStr + st * PAIR_BYTES;
                mbar_expect_tx(&x_full[st], PAIR_BYTES);
                if (DKV) {
                    const int i = fixed + n;
                    tma_load_4d(dst, &tmQKV, &x_full[st], 0, h, i * BT, b);                        // Q_i
                    tma_load_4d(dst + TILE_BYTES, &tmDO, &x_full[st], 0, h, i * BT, b);            // dO_i
                } else {
                    tma_load_4d(dst, &tmQKV, &x_full[st], 0, a.NH + h, n * BT, b);                 // K_j
                    tma_load_4d(dst + TILE_BYTES, &tmQKV, &x_full[st], 0, 2 * a.NH + h, n * BT, b);// V_j
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BT, 0, 0);
            constexpr uint32_t idesc_acc = DKV ? umma_idesc_bf16(BT, HS, 1, 1) : umma_idesc_bf16(BT, HS, 0, 1);
            auto issue_sdp = [&](int n) {
                const uint32_t xs = smem_u32(sStr + (n & 1) * PAIR_BYTES), rs = smem_u32(sRes);
                const uint32_t q = DKV ? xs : rs, dO = (DKV ? xs : rs) + TILE_BYTES;
                const uint32_t k = DKV ? rs : xs, v = (DKV ? rs : xs) + TILE_BYTES;
                #pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    umma_ss(tS, umma_desc_sw128(q + kk * 32, 16, 1024), umma_desc_sw128(k + kk * 32, 16, 1024), idesc_s, kk > 0);
                #pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    umma_ss(tdP, umma_desc_sw128(dO + kk * 32, 16, 1024), umma_desc_sw128(v + kk * 32, 16, 1024), idesc_s, kk > 0);
                umma_commit(sdp_full);
            };
            bool ok = mbar_wait(res_full, 0, abort_flag, a.status, 0x610);
            ok = ok && mbar_wait(&x_full[0], 0, abort_flag, a.status, 0x611);
            tc_fence_after();
            if (ok) issue_sdp(0);
            for (int n = 0; n < cnt && ok; n++) {
                if (n + 1 < cnt) {
                    if (!mbar_wait(&x_full[(n + 1) & 1], ((n + 1) >> 1) & 1, abort_flag, a.status, 0x612)) break;
                    if (!mbar_wait(sdp_empty, n & 1, abort_flag, a.status, 0x613)) break;
                    tc_fence_after();
                    issue_sdp(n + 1);
                }
                if (!mbar_wait(pds_full, n & 1, abort_flag, a.status, 0x614)) break;
                tc_fence_after();
                const uint32_t xs = smem_u32(sStr + (n & 1) * PAIR_BYTES), rs = smem_u32(sRes);
                const uint32_t p = smem_u32(sP), ds = smem_u32(sdS);
                if (DKV) {
                    // dV += P^T dO ; dK += dS^T Q : A is MN-major (two 64-wide groups 16 KB apart), K = 128 query rows
                    #pragma unroll
                    for (int kk = 0; kk < BT / 16; kk++)
                        umma_ss(tAcc0, umma_desc_sw128(p + kk * 2048, BT * 128, 1024), umma_desc_sw128(xs + TILE_BYTES + kk * 2048, 8192, 1024),
                                idesc_acc, (n > 0 || kk > 0));
                    #pragma unroll
                    for (int kk = 0; kk < BT / 16; kk++)
                        umma_ss(tAcc1, umma_desc_sw128(ds + kk * 2048, BT * 128, 1024), umma_desc_sw128(xs + kk * 2048, 8192, 1024),
                                idesc_acc, (n > 0 || kk > 0));
                } else {
                    // dQ += dS K : A K-major (two 64-column chunks), B = K_j as an N-major operand
                    #pragma unroll
                    for (int kk = 0; kk < BT / 16; kk++)
                        umma_ss(tAcc0, umma_desc_sw128(ds + (kk >> 2) * (BT * 128) + (kk & 3) * 32, 16, 1024),
                                umma_desc_sw128(xs + kk * 2048, 8192, 1024), idesc_acc, (n > 0 || kk > 0));
                }
                umma_commit(&x_empty[n & 1]);
                umma_commit(pds_empty);
                (void)rs;
            }
            umma_commit(acc_full);
        }
    } else {
        const int q = warp & 3;                        // TMEM lane quarter
        const int hf = (warp - 2) >> 2;                // column half handled by this thread
        const int r = q * 32 + lane;                   // row of the tile (a query row in S / dP)
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const float log2e = 1.4426950408889634f;
        const size_t stat_base = ((size_t)b * a.NH + h) * a.T;
        bool ok = true;
        for (int n = 0; n < cnt; n++) {
            const int qi = DKV ? fixed + n : fixed;    // query tile index
            const int kj = DKV ? fixed : n;            // key tile index
            const int t = qi * BT + r;
            float lse_l2 = 0.f, dlt = 0.f;
            const bool row_ok = t < a.T;
            if (row_ok) { lse_l2 = a.lse[stat_base + t] * log2e; dlt = a.delta[stat_base + t]; }
            ok = mbar_wait(sdp_full, n & 1, abort_flag, a.status, 0x620) && ok;
            tc_fence_after();
            uint32_t sv[64], dv[64];
            tmem_ld32(tS + lane_off + hf * 64, sv);
            tmem_ld32(tS + lane_off + hf * 64 + 32, sv + 32);
            tmem_ld32(tdP + lane_off + hf * 64, dv);
            tmem_ld32(tdP + lane_off + hf * 64 + 32, dv + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sdp_empty);      // S / dP may be overwritten by the next tile
            const bool diag = (qi == kj);
            uint32_t pp[32], dd[32];
            #pragma unroll
            for (int e = 0; e < 64; e += 2) {
                const int c0 = hf * 64 + e;
                float p0 = exp2f(__uint_as_float(sv[e]) * a.scale_log2e - lse_l2);
                float p1 = exp2f(__uint_as_float(sv[e + 1]) * a.scale_log2e - lse_l2);
                if (!row_ok || (diag && c0 > r)) p0 = 0.f;
                if (!row_ok || (diag && c0 + 1 > r)) p1 = 0.f;
                const float d0 = p0 * (__uint_as_float(dv[e]) - dlt) * a.scale;
                const float d1 = p1 * (__uint_as_float(dv[e + 1]) - dlt) * a.scale;
                pp[e >> 1] = pack_bf16x2(p0, p1);
                dd[e >> 1] = pack_bf16x2(d0, d1);
            }
            if (n > 0) ok = mbar_wait(pds_empty, (n - 1) & 1, abort_flag, a.status, 0x621) && ok;   // previous tile's MMAs have read P / dS
            uint8_t* prow = sP + hf * (BT * 128) + r * 128;
            uint8_t* drow = sdS + hf * (BT * 128) + r * 128;
            #pragma unroll
            for (int u = 0; u < 8; u++) {
                const int pos = (u ^ (r & 7)) * 16;
                if (DKV) *reinterpret_cast<uint4*>(prow + pos) = make_uint4(pp[u * 4], pp[u * 4 + 1], pp[u * 4 + 2], pp[u * 4 + 3]);
                *reinterpret_cast<uint4*>(drow + pos) = make_uint4(dd[u * 4], dd[u * 4 + 1], dd[u * 4 + 2], dd[u * 4 + 3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(pds_full);
        }
        ok = mbar_wait(acc_full, 0, abort_flag, a.status, 0x622) && ok;
        tc_fence_after();
        const int t = fixed * BT + r;
        {
            uint32_t v0[32];
            tmem_ld32(tAcc0 + lane_off + hf * 32, v0);
            tmem_ld_wait();
            if (t < a.T && ok) {
                // DKV: acc0 = dV (slot 2); else acc0 = dQ (slot 0)
                const int slot = DKV ? 2 : 0;
                bf16* dst = a.dqkv + (((size_t)b * a.T + t) * 3 + slot) * a.NH * HS + (size_t)h * HS + hf * 32;
                #pragma unroll
                for (int e = 0; e < 32; e += 8) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(v0[e]), __uint_as_float(v0[e + 1]));
                    o.y = pack_bf16x2(__uint_as_float(v0[e + 2]), __uint_as_float(v0[e + 3]));
                    o.z = pack_bf16x2(__uint_as_float(v0[e + 4]), __uint_as_float(v0[e + 5]));
                    o.w = pack_bf16x2(__uint_as_float(v0[e + 6]), __uint_as_float(v0[e + 7]));
                    *reinterpret_cast<uint4*>(dst + e) = o;
                }
            }
        }
        if (DKV) {
            uint32_t v1[32];
            tmem_ld32(tAcc1 + lane_off + hf * 32, v1);
            tmem_ld_wait();
            if (t < a.T && ok) {
                bf16* dst = a.dqkv + (((size_t)b * a.T + t) * 3 + 1) * a.NH * HS + (size_t)h * HS + hf * 32;   // dK
                #pragma unroll
                for (int e = 0; e < 32; e += 8) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(v1[e]), __uint_as_float(v1[e + 1]));
                    o.y = pack_bf16x2(__uint_as_float(v1[e + 2]), __uint_as_float(v1[e + 3]));
                    o.z = pack_bf16x2(__uint_as_float(v1[e + 4]), __uint_as_float(v1[e + 5]));
                    o.w = pack_bf16x2(__uint_as_float(v1[e + 6]), __uint_as_float(v1[e + 7]));
                    *reinterpret_cast<uint4*>(dst + e) = o;
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

// dqkv (B,T,3,NH,HS) = gradient of causal attention; delta: scratch of B*NH*T floats
extern "C" int llmc_attention_bwd(bf16* dqkv, float* delta, const bf16* dout, const bf16* qkv, const bf16* out, const float* lse,
                                  int B, int T, int NH, int hs, cudaStream_t stream) {
    if (hs != HS) { fprintf(stderr, "[llmc_b200] attention backward: head size %d not supported (64 only)\n", hs); return -1; }
    CUtensorMap tmQKV, tmDO;
    int rc = llmc_attn_qkv_map(&tmQKV, qkv, B, T, NH, hs);
    if (rc) return rc;
    {
        uint64_t dims[4] = {(uint64_t)hs, (uint64_t)NH, (uint64_t)T, (uint64_t)B};
        uint64_t strides[4] = {2, (uint64_t)hs * 2, (uint64_t)NH * hs * 2, (uint64_t)T * NH * hs * 2};
        uint32_t box[4] = {64, 1, 128, 1};
        if ((rc = llmc_get_tensormap(&tmDO, dout, 2, 4, dims, strides, box, 3))) return rc;
    }
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM));
        CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM));
        configured = true;
    }
    const long long rows = (long long)B * T * NH;
    delta_kernel<<<(unsigned)CEIL_DIV(rows * 8, 256), 256, 0, stream>>>(delta, out, dout, B, T, NH);
    CUDA_CHECK(cudaGetLastError());
    BwdArgs a;
    a.dqkv = dqkv; a.lse = lse; a.delta = delta; a.B = B; a.T = T; a.NH = NH;
    a.scale = 1.0f / sqrtf((float)hs);
    a.scale_log2e = a.scale * 1.4426950408889634f;
    a.status = llmc_status_ptr();
    const int nt = CEIL_DIV(T, BT);
    attn_bwd_kernel<true><<<B * NH * nt, BWD_THREADS, BWD_SMEM, stream>>>(tmQKV, tmDO, a);
    CUDA_CHECK(cudaGetLastError());
    attn_bwd_kernel<false><<<B * NH * nt, BWD_THREADS, BWD_SMEM, stream>>>(tmQKV, tmDO, a);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
