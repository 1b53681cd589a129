// Device-side building blocks shared by every sm_100a kernel in this library:
// 128-bit packed loads/stores, warp/block reductions, the SquirrelNoise5 stochastic
// rounding used for bf16 parameter updates, and thin wrappers around the Blackwell
// PTX this library is written against (mbarrier, TMA bulk tensor copies, tcgen05
// MMA / TMEM allocation / TMEM loads).
//
// Every wait on an mbarrier or on a flag written by another agent is bounded: after
// WAIT_LIMIT_CYCLES the waiter records an error code in a global status word, raises
// a CTA-wide abort flag that makes all later waits return immediately, and the kernel
// runs to its normal exit (freeing TMEM on the way).  The host reads the status word.
//
// Capability parity with llmc/cuda_common.h and llmc/cuda_utils.cuh of the reference
// (Packed128, warpReduce*, blockReduce, stochastic_rounding); the design is new.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>

typedef __nv_bfloat16 bf16;

#define DEVINL __device__ __forceinline__
#define CEIL_DIV(a, b) (((a) + (b) - 1) / (b))

// ----------------------------------------------------------------------------
// status word shared by all kernels of the library (see status.cu)
// 0 = ok. Non-zero = first error recorded: (code << 24) | detail
enum : unsigned int {
    ST_OK = 0,
    ST_MBAR_TIMEOUT = 1,   // a wait on a shared-memory mbarrier ran out
    ST_FLAG_TIMEOUT = 2,   // a wait on a global/peer flag ran out
    ST_BAD_ARG = 3,        // a kernel-side argument check failed
    ST_DEBUG_CHECK = 4,    // a check of the debug build failed (misaligned 16-byte access, id out of range); the access was skipped
};
extern "C" unsigned int* llmc_status_ptr();   // device pointer to the status word
extern "C" int llmc_device_sm_count();

// ----------------------------------------------------------------------------
// Checks of the debug build (-DLLMC_DEBUG_CHECKS, libllmc_b200_debug.so): a failed check records ST_DEBUG_CHECK with a
// location code in the status word and the kernel skips or clamps the access instead of faulting, so the context stays
// usable and the host sees which check fired.  In the normal build the macro is the constant true and costs nothing.
#ifdef LLMC_DEBUG_CHECKS
extern __device__ unsigned int* g_llmc_dbg_status;     // defined in runtime.cu (relocatable device code in the debug build)
__device__ __forceinline__ bool llmc_dbg_fail(unsigned int where) {
    if (g_llmc_dbg_status) atomicCAS(g_llmc_dbg_status, 0u, (4u << 24) | (where & 0xFFFFFFu));
    return false;
}
#define LLMC_DBG_CHECK(cond, where) ((cond) ? true : llmc_dbg_fail(where))
#else
#define LLMC_DBG_CHECK(cond, where) (true)
#endif
#define LLMC_ALIGNED16(p) ((reinterpret_cast<uintptr_t>(p) & 15u) == 0)

// ----------------------------------------------------------------------------
// 128-bit packs

template <typename T>
struct alignas(16) Pack128 {
    static constexpr int size = 16 / sizeof(T);
    T v[size];
    DEVINL T& operator[](int i) { return v[i]; }
    DEVINL const T& operator[](int i) const { return v[i]; }
    DEVINL static Pack128 zeros() {
        Pack128 p;
        #pragma unroll
        for (int i = 0; i < size; i++) p.v[i] = (T)0.0f;
        return p;
    }
};
typedef Pack128<bf16> bf16x8;
typedef Pack128<float> f32x4;

template <typename T> DEVINL Pack128<T> ld128(const T* p) {
    Pack128<T> r;
    if (!LLMC_DBG_CHECK(LLMC_ALIGNED16(p), 0xA10)) return Pack128<T>::zeros();
    *reinterpret_cast<int4*>(&r) = *reinterpret_cast<const int4*>(p); return r;
}
template <typename T> DEVINL Pack128<T> ld128cs(const T* p) {   // streaming: do not keep in L1
    Pack128<T> r;
    if (!LLMC_DBG_CHECK(LLMC_ALIGNED16(p), 0xA11)) return Pack128<T>::zeros();
    *reinterpret_cast<int4*>(&r) = __ldcs(reinterpret_cast<const int4*>(p)); return r;
}
template <typename T> DEVINL void st128(T* p, const Pack128<T>& v) {
    if (!LLMC_DBG_CHECK(LLMC_ALIGNED16(p), 0xA20)) return;
    *reinterpret_cast<int4*>(p) = *reinterpret_cast<const int4*>(&v);
}
template <typename T> DEVINL void st128cs(T* p, const Pack128<T>& v) {
    if (!LLMC_DBG_CHECK(LLMC_ALIGNED16(p), 0xA21)) return;
    __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}
template <typename T> DEVINL void st128cg(T* p, const Pack128<T>& v) {
    if (!LLMC_DBG_CHECK(LLMC_ALIGNED16(p), 0xA22)) return;
    __stcg(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}

DEVINL uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}
DEVINL float2 unpack_bf16x2(uint32_t u) {
    __nv_bfloat162 t = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(t);
}

// ----------------------------------------------------------------------------
// reductions

DEVINL float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
DEVINL float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum; every thread gets the result. `red` is >= 32 floats of shared memory.
DEVINL float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.0f;
    return warp_sum(r);
}
DEVINL float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    return warp_max(r);
}

// ----------------------------------------------------------------------------
// stochastic rounding fp32 -> bf16 (SquirrelNoise5 hash; same bit logic as the
// reference's llmc/cuda_utils.cuh:238-278 so that a checkpoint re-rounds identically)

DEVINL unsigned int squirrel_noise5(unsigned int position, unsigned int seed) {
    unsigned int m = position;
    m *= 0xd2a80a3fu; m += seed; m ^= (m >> 9);
    m += 0xa884f197u; m ^= (m >> 11);
    m *= 0x6C736F4Bu; m ^= (m >> 13);
    m += 0xB79F3ABBu; m ^= (m >> 15);
    m += 0x1b56c4f5u; m ^= (m >> 17);
    return m;
}
// `idx` is the logical noise index of the element's owner (see adamw.cu for the mapping)
DEVINL bf16 stochastic_round_bf16(float x, unsigned int noise) {
    unsigned int threshold = noise & 0xFFFFu;
    unsigned int bits = __float_as_uint(x);
    unsigned int rounded = ((bits & 0xFFFFu) > threshold) ? (bits | 0xFFFFu) : (bits & ~0xFFFFu);
    return __float2bfloat16_rn(__uint_as_float(rounded));
}

// ----------------------------------------------------------------------------
// math

DEVINL float gelu_tanh(float x) {
    const float k = 0.7978845608028654f;   // sqrt(2/pi)
    float c = x * x * x * 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k * (x + c)));
}
DEVINL float gelu_tanh_grad(float x) {
    const float k = 0.7978845608028654f;
    float c = x * x * x * 0.044715f;
    float t = tanhf(k * (x + c));
    float sech2 = 1.0f - t * t;
    return 0.5f * (1.0f + t) + x * 0.5f * sech2 * k * (1.0f + 3.0f * 0.044715f * x * x);
}

// The same functions on the hardware tanh approximation (MUFU, relative error about 2^-11, far below
// bf16 resolution).  Every device-side GELU in this library uses these, so a GELU output recomputed
// from a stored pre-activation is bit-identical to the one the GEMM epilogue produced.
// 2^x on the special-function unit (inputs here are <= 0 up to rounding, so no range handling is needed)
DEVINL float ex2_fast(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
DEVINL float tanh_fast(float x) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
DEVINL float gelu_fast(float x) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanh_fast(k * (x + 0.044715f * x * x * x)));
}
DEVINL float gelu_grad_fast(float x) {
    const float k = 0.7978845608028654f;
    const float x2 = x * x;
    const float t = tanh_fast(k * x * (1.0f + 0.044715f * x2));
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k * (1.0f + 3.0f * 0.044715f * x2);
}

// ----------------------------------------------------------------------------
// bounded waits

#ifndef WAIT_LIMIT_CYCLES
#define WAIT_LIMIT_CYCLES (3000000000ll)   // about 1.5 to 2.5 s at B200 clocks
#endif

DEVINL void record_error(unsigned int* status, unsigned int code, unsigned int detail) {
    if (status) atomicCAS(status, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

DEVINL void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
DEVINL void mbar_fence_init() {   // make inits visible to the async proxy / cluster
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
DEVINL void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
DEVINL void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DEVINL bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Wait for the phase with the given parity to complete. `abort_flag` is a CTA-shared
// word: once any waiter of the CTA has timed out, every wait returns at once.
// Returns false if the wait was abandoned.
DEVINL bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned int* status, unsigned int where) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            record_error(status, ST_MBAR_TIMEOUT, where);
            return false;
        }
    }
}

// try_wait with a suspend-time hint: the hardware parks the thread until the phase completes or about `ns` nanoseconds have
// passed, instead of the thread polling.
DEVINL bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// The same bounded wait for roles that wait long: each poll parks the thread in hardware (up to ~20 us), so the waiting warp takes
// no issue slots and makes no shared-memory traffic while it waits.
DEVINL bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned int* status, unsigned int where,
                              unsigned int unused = 0) {
    (void)unused;
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            record_error(status, ST_MBAR_TIMEOUT, where);
            return false;
        }
    }
}

// ----------------------------------------------------------------------------
// TMA (bulk tensor copies, never with cluster multicast)

DEVINL void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
DEVINL void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
DEVINL void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
DEVINL void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
DEVINL void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
DEVINL void tma_store_4d(const CUtensorMap* m, const void* smem_src, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
DEVINL void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> DEVINL void tma_store_wait_read() {   // smem of all but the N newest groups may be reused
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> DEVINL void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// generic-proxy writes to smem -> visible to the async proxy (before a TMA store / UMMA read)
DEVINL void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ----------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA, commit, TMEM loads

DEVINL void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
DEVINL void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
DEVINL void tmem_dealloc(uint32_t taddr, uint32_t ncols) {   // one full warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile.
//   lbo/sbo in bytes.  K-major: sbo = distance between 8-row groups (1024 when rows are
//   packed 128 B apart), lbo unused.  MN-major: lbo = distance between 64-element groups
//   along MN, sbo = distance between 8-row groups along K.
DEVINL uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;          // descriptor version of sm_100
    d |= (uint64_t)2 << 61;          // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16, bf16 x bf16 -> fp32
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread
DEVINL void umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
DEVINL void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on an mbarrier once all MMAs issued so far by this thread have completed
DEVINL void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base_lane + i), columns c..c+31
DEVINL void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
DEVINL void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
DEVINL void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 columns store (registers -> TMEM)
DEVINL void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
DEVINL void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

DEVINL bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------
// host-side helpers (tensor maps); implemented in tensormap.cu
#define CUDA_CHECK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
    fprintf(stderr, "[llmc_b200] CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); return (int)e_; } } while (0)
// Encode (or fetch from a cache) a tiled tensor map over bf16/fp32 data.
//  rank 2..4; dims/strides innermost first (strides in bytes, strides[0] implied = elem size)
//  swizzle: 0 none, 1 = 32B, 2 = 64B, 3 = 128B
int llmc_get_tensormap(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, int swizzle);
