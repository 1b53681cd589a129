// Causal flash attention forward for sm_100a on the packed (B, T, 3, NH, HS) QKV layout, HS = 64.
//
// One CTA per (batch, head, 128-row query tile); two CTAs share an SM so that one CTA's softmax
// overlaps the other's tensor-core work.  Roles inside a CTA (192 threads):
//   warp 0     TMA producer: Q once, then K tiles (double buffered) and V tiles (single buffer),
//              read in place from the packed QKV tensor through a 4-D tensor map.
//   warp 1     MMA issuer: S = Q K^T into TMEM columns [0,128), PV = P V into TMEM columns [128,192).
//   warps 2-5  softmax: thread r owns query row r.  Two passes over the S row in TMEM (max, then
//              exp / row sum / bf16 P written to 128-byte-swizzled shared memory as the A operand of
//              the PV MMA); the output row lives in 64 fp32 registers and is rescaled on line.
// Statistics are written as natural-log LSE per (b, h, t), the layout cuDNN's SDPA uses in the
// reference (llmc/cudnn_att.cpp:105-113).  Tiles above the diagonal are skipped.
//
// Capability parity: attention_forward_cudnn (llmc/cudnn_att.cpp:222-254) and the unfused
// attention_forward of llmc/attention.cuh in the reference.
#include "common.cuh"

namespace {

constexpr int HS = 64;
constexpr int BQ = 128, BKV = 128;
constexpr int TILE_BYTES = 128 * HS * 2;           // 16 KB: a 128 x 64 bf16 tile
constexpr int P_BYTES = BQ * BKV * 2;              // 32 KB
constexpr int FWD_SMEM = TILE_BYTES /*Q*/ + 2 * TILE_BYTES /*K*/ + TILE_BYTES /*V*/ + P_BYTES + 256;
constexpr int FWD_THREADS = 192;
constexpr int FWD_TMEM_COLS = 256;

struct FwdArgs {
    bf16* out;         // (B, T, NH, HS)
    float* lse;        // (B, NH, T)
    int B, T, NH;
    float scale_log2e; // (1/sqrt(HS)) * log2(e)
    float scale;
    unsigned int* status;
};

__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const FwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + TILE_BYTES;             // 2 stages
    uint8_t* sV = sK + 2 * TILE_BYTES;
    uint8_t* sP = sV + TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;     // [2]
    uint64_t* k_empty = bars + 3;    // [2]
    uint64_t* v_full = bars + 5;
    uint64_t* s_full = bars + 6;
    uint64_t* s_empty = bars + 7;
    uint64_t* p_full = bars + 8;
    uint64_t* o_full = bars + 9;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nq = CEIL_DIV(a.T, BQ);
    // heavy (late) query tiles first
    const int qi = nq - 1 - (int)(blockIdx.x / (a.B * a.NH));
    const int bh = blockIdx.x % (a.B * a.NH);
    const int b = bh / a.NH, h = bh % a.NH;
    const int n_kv = qi + 1;

    if (threadIdx.x == 0) {
        if ((smem_u32(smem) & 1023u) != 0) record_error(a.status, ST_BAD_ARG, 0x10);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
        mbar_init(v_full, 1); mbar_init(s_full, 1); mbar_init(s_empty, 4); mbar_init(p_full, 4); mbar_init(o_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, FWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tO = tmem_base + 128;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_4d(sQ, &tmQKV, q_full, 0, h, qi * BQ, b);
            for (int j = 0; j < n_kv; j++) {
                const int st = j & 1;
                if (!mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, a.status, 0x500)) break;
                mbar_expect_tx(&k_full[st], TILE_BYTES);
                tma_load_4d(sK + st * TILE_BYTES, &tmQKV, &k_full[st], 0, a.NH + h, j * BKV, b);
                if (j > 0) { if (!mbar_wait(o_full, (j - 1) & 1, abort_flag, a.status, 0x501)) break; }   // PV(j-1) has read V
                mbar_expect_tx(v_full, TILE_BYTES);
                tma_load_4d(sV, &tmQKV, v_full, 0, 2 * a.NH + h, j * BKV, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, 0, 0);     // Q (K-major) x K (K-major)
            constexpr uint32_t idesc_o = umma_idesc_bf16(BQ, HS, 0, 1);      // P (K-major) x V (N-major)
            auto issue_s = [&](int j) {
                const uint32_t q = smem_u32(sQ), k = smem_u32(sK + (j & 1) * TILE_BYTES);
                #pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    umma_ss(tS, umma_desc_sw128(q + kk * 32, 16, 1024), umma_desc_sw128(k + kk * 32, 16, 1024), idesc_s, kk > 0);
                umma_commit(s_full);
                umma_commit(&k_empty[j & 1]);
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, a.status, 0x510);
            ok = ok && mbar_wait(&k_full[0], 0, abort_flag, a.status, 0x511);
            tc_fence_after();
            if (ok) issue_s(0);
            for (int j = 0; j < n_kv && ok; j++) {
                if (j + 1 < n_kv) {
                    if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag, a.status, 0x512)) break;
                    if (!mbar_wait(s_empty, j & 1, abort_flag, a.status, 0x513)) break;
                    tc_fence_after();
                    issue_s(j + 1);
                }
                if (!mbar_wait(p_full, j & 1, abort_flag, a.status, 0x514)) break;
                if (!mbar_wait(v_full, j & 1, abort_flag, a.status, 0x515)) break;
                tc_fence_after();
                const uint32_t p = smem_u32(sP), v = smem_u32(sV);
                #pragma unroll
                for (int kk = 0; kk < BKV / 16; kk++) {
                    // P: two 64-column swizzled chunks of 16 KB; V: 128 kv rows of 128 B, 16 rows per K step
                    const uint32_t pa = p + (kk >> 2) * (BQ * 128) + (kk & 3) * 32;
                    umma_ss(tO, umma_desc_sw128(pa, 16, 1024), umma_desc_sw128(v + kk * 2048, 8192, 1024), idesc_o, kk > 0);
                }
                umma_commit(o_full);
            }
        }
    } else {
        const int q = warp & 3;
        const int r = q * 32 + lane;                 // query row inside the tile
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        float m = -INFINITY, l = 0.f;
        float O[HS];
        #pragma unroll
        for (int d = 0; d < HS; d++) O[d] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv; j++) {
            ok = mbar_wait(s_full, j & 1, abort_flag, a.status, 0x520) && ok;
            tc_fence_after();
            const bool diag = (j == qi);
            // pass 1: row maximum
            float mx = m;
            #pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tS + lane_off + c * 32, v);
                tmem_ld_wait();
                #pragma unroll
                for (int e = 0; e < 32; e++) {
                    float s = __uint_as_float(v[e]);
                    if (diag && (c * 32 + e > r)) s = -INFINITY;
                    mx = fmaxf(mx, s);
                }
            }
            const float alpha = exp2f((m - mx) * a.scale_log2e);     // m = -inf on the first tile -> 0
            m = mx;
            const float moff = m * a.scale_log2e;
            // fold in the previous tile's P V (its MMA finished while we were waiting for S)
            if (j > 0) {
                ok = mbar_wait(o_full, (j - 1) & 1, abort_flag, a.status, 0x521) && ok;
                tc_fence_after();
                #pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t v[32];
                    tmem_ld32(tO + lane_off + c * 32, v);
                    tmem_ld_wait();
                    #pragma unroll
                    for (int e = 0; e < 32; e++) O[c * 32 + e] += __uint_as_float(v[e]);
                }
            }
            #pragma unroll
            for (int d = 0; d < HS; d++) O[d] *= alpha;
            l *= alpha;
            // pass 2: probabilities -> bf16 P in shared memory (A operand of the P V MMA)
            float rs = 0.f;
            #pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tS + lane_off + c * 32, v);
                tmem_ld_wait();
                uint32_t pk[16];
                #pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0 = exp2f(__uint_as_float(v[e]) * a.scale_log2e - moff);
                    float p1 = exp2f(__uint_as_float(v[e + 1]) * a.scale_log2e - moff);
                    if (diag && (c * 32 + e > r)) p0 = 0.f;
                    if (diag && (c * 32 + e + 1 > r)) p1 = 0.f;
                    rs += p0 + p1;
                    pk[e >> 1] = pack_bf16x2(p0, p1);
                }
                uint8_t* prow = sP + (c >> 1) * (BQ * 128) + r * 128;
                #pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int unit = (c & 1) * 4 + u;      // 16-byte unit inside the 128-byte row
                    *reinterpret_cast<uint4*>(prow + ((unit ^ (r & 7)) * 16)) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
                }
            }
            l += rs;
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(s_empty); mbar_arrive(p_full); }
        }
        ok = mbar_wait(o_full, (n_kv - 1) & 1, abort_flag, a.status, 0x522) && ok;
        tc_fence_after();
        #pragma unroll
        for (int c = 0; c < 2; c++) {
            uint32_t v[32];
            tmem_ld32(tO + lane_off + c * 32, v);
            tmem_ld_wait();
            #pragma unroll
            for (int e = 0; e < 32; e++) O[c * 32 + e] += __uint_as_float(v[e]);
        }
        const int t = qi * BQ + r;
        if (t < a.T && ok) {
            const float inv = 1.0f / l;
            bf16* op = a.out + (((size_t)b * a.T + t) * a.NH + h) * HS;
            #pragma unroll
            for (int d = 0; d < HS; d += 8) {
                uint4 o;
                o.x = pack_bf16x2(O[d] * inv, O[d + 1] * inv); o.y = pack_bf16x2(O[d + 2] * inv, O[d + 3] * inv);
                o.z = pack_bf16x2(O[d + 4] * inv, O[d + 5] * inv); o.w = pack_bf16x2(O[d + 6] * inv, O[d + 7] * inv);
                *reinterpret_cast<uint4*>(op + d) = o;
            }
            a.lse[((size_t)b * a.NH + h) * a.T + t] = m * a.scale + logf(l);
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
    if (warp == 1) tmem_dealloc(tmem_base, FWD_TMEM_COLS);
}

}  // namespace

// Tensor map over a packed (B, T, 3, NH, HS) tensor seen as 4-D {HS, 3*NH, T, B} with a 128-row box.
int llmc_attn_qkv_map(CUtensorMap* tm, const bf16* qkv, int B, int T, int NH, int hs) {
    uint64_t dims[4] = {(uint64_t)hs, (uint64_t)(3 * NH), (uint64_t)T, (uint64_t)B};
    uint64_t strides[4] = {2, (uint64_t)hs * 2, (uint64_t)3 * NH * hs * 2, (uint64_t)T * 3 * NH * hs * 2};
    uint32_t box[4] = {64, 1, 128, 1};
    return llmc_get_tensormap(tm, qkv, 2, 4, dims, strides, box, 3);
}

// out (B,T,NH,HS) = causal softmax(Q K^T / sqrt(HS)) V ; lse (B,NH,T) fp32
extern "C" int llmc_attention_fwd(bf16* out, float* lse, const bf16* qkv, int B, int T, int NH, int hs, cudaStream_t stream) {
    if (hs != HS) { fprintf(stderr, "[llmc_b200] attention: head size %d not supported (64 only)\n", hs); return -1; }
    CUtensorMap tm;
    int rc = llmc_attn_qkv_map(&tm, qkv, B, T, NH, hs);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
        configured = true;
    }
    FwdArgs a;
    a.out = out; a.lse = lse; a.B = B; a.T = T; a.NH = NH;
    a.scale = 1.0f / sqrtf((float)hs);
    a.scale_log2e = a.scale * 1.4426950408889634f;
    a.status = llmc_status_ptr();
    const int nq = CEIL_DIV(T, BQ);
    attn_fwd_kernel<<<B * NH * nq, FWD_THREADS, FWD_SMEM, stream>>>(tm, a);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
