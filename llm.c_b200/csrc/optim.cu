// Optimizer-side kernels on flat parameter / gradient buffers: squared global gradient norm,
// AdamW with fp32 master weights and stochastic rounding to bf16, re-rounding of parameters from the
// master copy (resume), master initialisation from bf16 parameters.
//
// All kernels take a table of up to 16 "tensor views".  A view describes the part of one parameter
// tensor this rank owns: `L` layer slices of `n` elements each, slice l starting at
// p_base + l * p_stride in the parameter/gradient buffers and at o_base + l * o_stride in the
// optimizer-state buffers (m, v, master).  With one rank the views cover whole tensors; with ZeRO-1
// they cover this rank's 1/N of every layer slice, which is the layout the reference stores in its
// state files (train_gpt2.cu:1035-1124 of the reference).
//
// The clipping coefficient is computed on the device from the squared norm, so a training step
// needs no host synchronisation between backward and the parameter update.
//
// Capability parity: llmc/adamw.cuh, llmc/global_norm.cuh, init_from_master, copy_and_cast.
#include "common.cuh"

struct TensorView {
    long long p_base, p_stride, o_base, o_stride, n;
    int L;
    float wd;              // weight decay applied to this tensor
    unsigned int seed;     // stochastic rounding seed of this tensor for this step
    int pad;
};
struct TensorTable {
    TensorView t[16];
    int count;
};

namespace {

constexpr int OPT_THREADS = 512;

__global__ void __launch_bounds__(OPT_THREADS)
norm_sq_kernel(float* __restrict__ partials, const bf16* __restrict__ grads, const TensorTable tab) {
    __shared__ float red[32];
    const TensorView tv = tab.t[blockIdx.y];
    const long long packs_per_slice = tv.n >> 3;
    // slice by slice (no division per pack), four independent 128-bit loads in flight per thread; the order of the additions is
    // fixed by the launch geometry, which the host derives from the device alone: the same sum on every run
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    const long long stride = (long long)gridDim.x * OPT_THREADS;
    for (int l = 0; l < tv.L; l++) {
        const bf16* base = grads + tv.p_base + (long long)l * tv.p_stride;
        long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x;
        for (; i + 3 * stride < packs_per_slice; i += 4 * stride) {
            const bf16x8 g0 = ld128cs(base + i * 8), g1 = ld128cs(base + (i + stride) * 8), g2 = ld128cs(base + (i + 2 * stride) * 8),
                         g3 = ld128cs(base + (i + 3 * stride) * 8);
            #pragma unroll
            for (int e = 0; e < 8; e++) {
                const float f0 = __bfloat162float(g0[e]), f1 = __bfloat162float(g1[e]), f2 = __bfloat162float(g2[e]), f3 = __bfloat162float(g3[e]);
                a0 = fmaf(f0, f0, a0); a1 = fmaf(f1, f1, a1); a2 = fmaf(f2, f2, a2); a3 = fmaf(f3, f3, a3);
            }
        }
        for (; i < packs_per_slice; i += stride) {
            const bf16x8 g = ld128cs(base + i * 8);
            #pragma unroll
            for (int e = 0; e < 8; e++) { const float f = __bfloat162float(g[e]); a0 = fmaf(f, f, a0); }
        }
    }
    float acc = (a0 + a1) + (a2 + a3);
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) partials[blockIdx.y * gridDim.x + blockIdx.x] = acc;
}

// out[0] = scale * sum(partials[0..n)) in index order with a fixed tree: deterministic
__global__ void __launch_bounds__(1024) final_sum_kernel(float* __restrict__ out, const float* __restrict__ partials, int n, float scale = 1.0f) {
    __shared__ float red[32];
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += 1024) acc += partials[i];
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) out[0] = acc * scale;
}

DEVINL unsigned int sr_position(long long idx, int layer) {
    // noise index of element `idx` of layer slice `layer`; a pure function of the element, so the
    // result does not depend on launch geometry (needed for bit-exact resume from a state file)
    return (unsigned int)(idx & 511) + 198491317u * ((unsigned int)(idx & ~511ll) + (unsigned int)layer);
}

template <bool HAS_MASTER>
__global__ void __launch_bounds__(OPT_THREADS)
adamw_kernel(bf16* __restrict__ params, float* __restrict__ master, const bf16* __restrict__ grads,
             float* __restrict__ m_buf, float* __restrict__ v_buf, const TensorTable tab,
             float lr, float beta1, float beta2, float bc1, float bc2, float eps,
             float grad_scale, const float* __restrict__ norm_sq, float grad_clip) {
    float scale = grad_scale;
    if (norm_sq != nullptr) {
        const float nsq = norm_sq[0];
        if (!(nsq >= 0.f) || isinf(nsq)) return;          // non-finite gradient: skip the whole update
        const float nrm = sqrtf(nsq);
        scale = (nrm > grad_clip) ? grad_scale * grad_clip / nrm : grad_scale;
    }
    const TensorView tv = tab.t[blockIdx.y];
    const long long total = tv.n * tv.L;
    for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * OPT_THREADS) {
        const long long l = i / tv.n, idx = i - l * tv.n;
        const long long pi = tv.p_base + l * tv.p_stride + idx;
        const long long oi = tv.o_base + l * tv.o_stride + idx;
        const float g = scale * __bfloat162float(grads[pi]);
        float m = m_buf[oi], v = v_buf[oi];
        m = fmaf(beta1, m, (1.0f - beta1) * g);          // lerp(g, m, beta1)
        v = fmaf(beta2, v, (1.0f - beta2) * g * g);
        m_buf[oi] = m; v_buf[oi] = v;
        const float mh = m / bc1, vh = v / bc2;
        const float old = HAS_MASTER ? master[oi] : __bfloat162float(params[pi]);
        const float p = old - lr * (mh / (sqrtf(vh) + eps) + tv.wd * old);
        params[pi] = stochastic_round_bf16(p, squirrel_noise5(sr_position(idx, (int)l + tv.pad), tv.seed));
        if (HAS_MASTER) master[oi] = p;
    }
}

// The same update on 8-element packs (128-bit accesses): every tensor slice of a transformer is a multiple of 8 elements, and so
// are its ZeRO shards (the sharding rule demands it); the element-wise kernel above stays as the fallback for odd layouts.
template <bool HAS_MASTER>
__global__ void __launch_bounds__(OPT_THREADS)
adamw_pack_kernel(bf16* __restrict__ params, float* __restrict__ master, const bf16* __restrict__ grads,
                  float* __restrict__ m_buf, float* __restrict__ v_buf, const TensorTable tab,
                  float lr, float beta1, float beta2, float bc1, float bc2, float eps,
                  float grad_scale, const float* __restrict__ norm_sq, float grad_clip) {
    float scale = grad_scale;
    if (norm_sq != nullptr) {
        const float nsq = norm_sq[0];
        if (!(nsq >= 0.f) || isinf(nsq)) return;          // non-finite gradient: skip the whole update
        const float nrm = sqrtf(nsq);
        scale = (nrm > grad_clip) ? grad_scale * grad_clip / nrm : grad_scale;
    }
    const TensorView tv = tab.t[blockIdx.y];
    const long long packs_per_slice = tv.n >> 3;
    const long long total = packs_per_slice * tv.L;
    for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * OPT_THREADS) {
        const long long l = i / packs_per_slice, pk = i - l * packs_per_slice;
        const long long pi = tv.p_base + l * tv.p_stride + pk * 8;
        const long long oi = tv.o_base + l * tv.o_stride + pk * 8;
        const bf16x8 g = ld128cs(grads + pi);
        f32x4 m0 = ld128cs(m_buf + oi), m1 = ld128cs(m_buf + oi + 4), v0 = ld128cs(v_buf + oi), v1 = ld128cs(v_buf + oi + 4);
        f32x4 w0, w1;
        if (HAS_MASTER) { w0 = ld128cs(master + oi); w1 = ld128cs(master + oi + 4); }
        else {
            const bf16x8 pw = ld128(params + pi);
            #pragma unroll
            for (int e = 0; e < 4; e++) { w0[e] = __bfloat162float(pw[e]); w1[e] = __bfloat162float(pw[e + 4]); }
        }
        bf16x8 out;
        #pragma unroll
        for (int e = 0; e < 8; e++) {
            float& mm = e < 4 ? m0[e] : m1[e - 4];
            float& vv = e < 4 ? v0[e] : v1[e - 4];
            float& ww = e < 4 ? w0[e] : w1[e - 4];
            const float gg = scale * __bfloat162float(g[e]);
            mm = fmaf(beta1, mm, (1.0f - beta1) * gg);
            vv = fmaf(beta2, vv, (1.0f - beta2) * gg * gg);
            // the same expressions as the element-wise kernel (division by the bias corrections included), so both give the same bits
            const float mh = mm / bc1, vh = vv / bc2;
            ww = ww - lr * (mh / (sqrtf(vh) + eps) + tv.wd * ww);
            out[e] = stochastic_round_bf16(ww, squirrel_noise5(sr_position(pk * 8 + e, (int)l + tv.pad), tv.seed));
        }
        st128cs(m_buf + oi, m0); st128cs(m_buf + oi + 4, m1); st128cs(v_buf + oi, v0); st128cs(v_buf + oi + 4, v1);
        if (HAS_MASTER) { st128cs(master + oi, w0); st128cs(master + oi + 4, w1); }
        st128(params + pi, out);
    }
}

// params <- stochastic_round(master) with the given seeds (resume path)
__global__ void __launch_bounds__(OPT_THREADS)
from_master_kernel(bf16* __restrict__ params, const float* __restrict__ master, const TensorTable tab) {
    const TensorView tv = tab.t[blockIdx.y];
    const long long total = tv.n * tv.L;
    for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * OPT_THREADS) {
        const long long l = i / tv.n, idx = i - l * tv.n;
        params[tv.p_base + l * tv.p_stride + idx] =
            stochastic_round_bf16(master[tv.o_base + l * tv.o_stride + idx], squirrel_noise5(sr_position(idx, (int)l + tv.pad), tv.seed));
    }
}

// master <- float(params)
__global__ void __launch_bounds__(OPT_THREADS)
to_master_kernel(float* __restrict__ master, const bf16* __restrict__ params, const TensorTable tab) {
    const TensorView tv = tab.t[blockIdx.y];
    const long long total = tv.n * tv.L;
    for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * OPT_THREADS) {
        const long long l = i / tv.n, idx = i - l * tv.n;
        master[tv.o_base + l * tv.o_stride + idx] = __bfloat162float(params[tv.p_base + l * tv.p_stride + idx]);
    }
}

int opt_grid_x() { int sms = llmc_device_sm_count(); if (sms <= 0) sms = 148; return sms; }

}  // namespace

// out[0] = scale * sum of n floats, one block, fixed summation tree (the mean loss of a step; reference:
// global_sum_deterministic, llmc/cuda_utils.cuh:188-206)
extern "C" int llmc_sum_f32(float* out, const float* in, int n, float scale, cudaStream_t stream) {
    final_sum_kernel<<<1, 1024, 0, stream>>>(out, in, n, scale);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_norm_sq_scratch() { return 16 * opt_grid_x(); }

// out[0] = sum of squares of the gradient elements covered by the table. `partials`: llmc_norm_sq_scratch floats.
extern "C" int llmc_global_norm_sq(float* out, float* partials, const bf16* grads, const TensorTable* tab, cudaStream_t stream) {
    const int gx = opt_grid_x();
    for (int i = 0; i < tab->count; i++) if (tab->t[i].n % 8 || tab->t[i].p_base % 8 || tab->t[i].p_stride % 8) return -1;
    norm_sq_kernel<<<dim3(gx, tab->count), OPT_THREADS, 0, stream>>>(partials, grads, *tab);
    CUDA_CHECK(cudaGetLastError());
    final_sum_kernel<<<1, 1024, 0, stream>>>(out, partials, gx * tab->count);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

// One AdamW step over the views of the table. t = step number starting at 1.
// If norm_sq (device pointer) is given, the gradient is additionally scaled by
// min(1, grad_clip / sqrt(norm_sq[0])) and the update is skipped if norm_sq is not finite.
extern "C" int llmc_adamw(bf16* params, float* master, const bf16* grads, float* m, float* v, const TensorTable* tab,
                          float lr, float beta1, float beta2, float eps, int t, float grad_scale,
                          const float* norm_sq, float grad_clip, cudaStream_t stream) {
    const float bc1 = 1.0f - powf(beta1, (float)t), bc2 = 1.0f - powf(beta2, (float)t);
    dim3 grid(opt_grid_x() * 2, tab->count);
    bool packs = true;
    for (int i = 0; i < tab->count; i++) {
        const TensorView& tv = tab->t[i];
        if (tv.n % 8 || tv.p_base % 8 || tv.p_stride % 8 || tv.o_base % 8 || tv.o_stride % 8) packs = false;
    }
    if (packs) {
        if (master) adamw_pack_kernel<true><<<grid, OPT_THREADS, 0, stream>>>(params, master, grads, m, v, *tab, lr, beta1, beta2, bc1, bc2, eps, grad_scale, norm_sq, grad_clip);
        else adamw_pack_kernel<false><<<grid, OPT_THREADS, 0, stream>>>(params, master, grads, m, v, *tab, lr, beta1, beta2, bc1, bc2, eps, grad_scale, norm_sq, grad_clip);
    } else if (master) adamw_kernel<true><<<grid, OPT_THREADS, 0, stream>>>(params, master, grads, m, v, *tab, lr, beta1, beta2, bc1, bc2, eps, grad_scale, norm_sq, grad_clip);
    else adamw_kernel<false><<<grid, OPT_THREADS, 0, stream>>>(params, master, grads, m, v, *tab, lr, beta1, beta2, bc1, bc2, eps, grad_scale, norm_sq, grad_clip);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_params_from_master(bf16* params, const float* master, const TensorTable* tab, cudaStream_t stream) {
    from_master_kernel<<<dim3(opt_grid_x() * 2, tab->count), OPT_THREADS, 0, stream>>>(params, master, *tab);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int llmc_master_from_params(float* master, const bf16* params, const TensorTable* tab, cudaStream_t stream) {
    to_master_kernel<<<dim3(opt_grid_x() * 2, tab->count), OPT_THREADS, 0, stream>>>(master, params, *tab);
    CUDA_CHECK(cudaGetLastError());
    return 0;
}
