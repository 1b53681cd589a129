// TF32 GEMM for the full-precision mode: D[M,N] (+)= A[M,K] * B[N,K]^T (+ bias), fp32 in memory, tcgen05.mma kind::tf32
// with fp32 accumulation in TMEM.
//
// The full-precision mode keeps every tensor in fp32 (the counterpart of the reference's train_gpt2_fp32.cu and of its
// PRECISION=FP32 build, where cuBLAS runs the matmuls in TF32 when -f 1).  Both operands are K-major ("TN"): the forward
// product reads them as stored; the operator layer hands transposed copies for the two backward products.
//
// Structure of a CTA (192 threads, persistent, tiles taken round-robin):
//   warp 0      TMA producer: 4-stage ring of 128 x 32 fp32 tiles of A and of B (128-byte rows, 128-byte swizzle)
//   warp 1      MMA issuer: four tcgen05.mma 128 x 128 x 8 per stage into one of two 128-column TMEM accumulators
//   warps 2..5  epilogue: thread = one row; tcgen05.ld 32 columns at a time, add the bias or the previous contents of D,
//               write 128 contiguous bytes per thread with 16-byte stores
// No TMA load uses cluster multicast.  All waits are bounded (see common.cuh).
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 4;      // BK fp32 = 128 bytes
constexpr int UMMA_K = 8;                                    // tf32: 32 bytes of K per instruction
constexpr int A_STAGE_BYTES = BM * BK * 4;                   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 4;                   // 16 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int RASTER_GROUP = 16;

struct Tf32Args {
    int M, N, K;
    int num_m_tiles, num_n_tiles, num_kb;
    float* D; int ldd;
    const float* bias;      // N entries or null
    int accumulate;         // add to the existing D
    unsigned int* status;
};

// Instruction descriptor, kind::tf32: fp32 accumulator (bit 4), A and B formats TF32 (value 2 at bits 7 and 10), both K-major
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
DEVINL void umma_ss_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Tf32Args g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                    // [STAGES]
    uint64_t* empty = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_work = g.num_m_tiles * g.num_n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // m tiles are visited in groups so that concurrently running CTAs share both A and B tiles in L2
    auto decode = [&](int w, int& mt, int& nt) {
        const int per_group = RASTER_GROUP * g.num_n_tiles;
        const int grp = w / per_group, within = w - grp * per_group;
        const int gh = min(RASTER_GROUP, g.num_m_tiles - grp * RASTER_GROUP);
        nt = within / gh;
        mt = grp * RASTER_GROUP + within - nt * gh;
    };

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
                int mt, nt; decode(w, mt, nt);
                for (int kb = 0; kb < g.num_kb; kb++) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, g.status, 0xD00 + stage)) break;
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    mbar_expect_tx(&full[stage], STAGE_BYTES);
                    tma_load_2d(sa, &tmA, &full[stage], kb * BK, mt * BM);                       // box {32 k, 128 rows}
                    tma_load_2d(sa + A_STAGE_BYTES, &tmB, &full[stage], kb * BK, nt * BN);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (*abort_flag) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_tf32(BM, BN);
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            for (int w = blockIdx.x; w < total_work; w += gridDim.x, it++) {
                const int buf = it & 1;
                const uint32_t use = (uint32_t)(it >> 1);
                if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, g.status, 0xD10 + buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < g.num_kb; kb++) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, g.status, 0xD20 + stage)) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    #pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)          // 8 fp32 of K = 32 bytes inside the swizzled 128-byte row
                        umma_ss_tf32(d_tmem, umma_desc_sw128(sa + k * 32, 16, 1024), umma_desc_sw128(sb + k * 32, 16, 1024), idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                umma_commit(&acc_full[buf]);
                if (*abort_flag) break;
            }
        }
    } else {
        const int q = warp & 3;                        // TMEM lane quarter this warp may access
        const int row = q * 32 + lane;
        int it = 0;
        for (int w = blockIdx.x; w < total_work; w += gridDim.x, it++) {
            int mt, nt; decode(w, mt, nt);
            const int buf = it & 1;
            const uint32_t use = (uint32_t)(it >> 1);
            const bool ok = mbar_wait(&acc_full[buf], use & 1, abort_flag, g.status, 0xD30 + buf);
            tc_fence_after();
            const int grow = mt * BM + row;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            #pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                const int col0 = nt * BN + c * 32;
                if (col0 >= g.N) break;
                uint32_t v[32];
                tmem_ld32(t_row + c * 32, v);
                tmem_ld_wait();
                if (grow < g.M && ok) {
                    float* dp = g.D + (size_t)grow * g.ldd + col0;
                    #pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        if (col0 + j < g.N) {                     // N is a multiple of 4
                            float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                            if (g.bias != nullptr) {
                                const float4 b = *reinterpret_cast<const float4*>(g.bias + col0 + j);
                                o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                            }
                            if (g.accumulate) {
                                const float4 old = *reinterpret_cast<const float4*>(dp + j);
                                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            }
                            *reinterpret_cast<float4*>(dp + j) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (*abort_flag) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {                                 // give loads in flight time to land before the CTA's memory goes away
        long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace

// D[M,N] (+)= A[M,K] * B[N,K]^T (+ bias[N]); all fp32, row-major with leading dimensions in elements.
// K, N and the leading dimensions must be multiples of 4 (16-byte rows for TMA and for the vector stores).
extern "C" int llmc_gemm_tf32(const float* A, const float* B, float* D, const float* bias, int M, int N, int K, int lda, int ldb, int ldd,
                              int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((N % 4) || (K % 4) || (lda % 4) || (ldb % 4) || (ldd % 4)) return -1;
    Tf32Args g;
    g.M = M; g.N = N; g.K = K;
    g.num_m_tiles = CEIL_DIV(M, BM); g.num_n_tiles = CEIL_DIV(N, BN); g.num_kb = CEIL_DIV(K, BK);
    g.D = D; g.ldd = ldd; g.bias = bias; g.accumulate = accumulate;
    g.status = llmc_status_ptr();
    CUtensorMap tmA, tmB;
    int rc;
    {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[2] = {4, (uint64_t)lda * 4};
        uint32_t box[2] = {BK, BM};
        if ((rc = llmc_get_tensormap(&tmA, A, 4, 2, dims, strides, box, 3))) return rc;
    }
    {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)N}, strides[2] = {4, (uint64_t)ldb * 4};
        uint32_t box[2] = {BK, BN};
        if ((rc = llmc_get_tensormap(&tmB, B, 4, 2, dims, strides, box, 3))) return rc;
    }
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(gemm_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148;
    const int total = g.num_m_tiles * g.num_n_tiles;
    const int grid = total < sms ? total : sms;
    gemm_tf32_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, g);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
