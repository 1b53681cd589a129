"""Thin launchers of the sm_100a kernels: tensors in, C entry points out (see csrc/*.cu)."""
import ctypes
import os

import torch

from .. import _lib
from .._lib import TensorTable, check

MODE_STORE, MODE_GELU, MODE_DGELU, MODE_ACCUM = 0, 1, 2, 3

_launches = 0   # number of kernel-library launches issued (bench.py reports it)
# forward / dgrad GEMMs with at least this many 256 x 256 tiles run on the two-SM kernel (gemm2.cu); 0 disables it
TWO_SM_MIN_TILES = int(os.environ.get("LLMC_GEMM_2SM_MIN_TILES", "74"))


def launch_count():
    return _launches


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


class _Scratch:
    """Per-device scratch buffers that grow to the largest request and are then reused."""

    def __init__(self):
        self.bufs = {}

    def get(self, key, numel, dtype, device, zero=False):
        k = (key, device.index, dtype)
        t = self.bufs.get(k)
        if t is None or t.numel() < numel:
            t = (torch.zeros if zero else torch.empty)(max(int(numel), 1), dtype=dtype, device=device)
            self.bufs[k] = t
        return t


_scratch = _Scratch()
_sm_count = {}


def sm_count(device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def gemm(a, b, d, M, N, K, lda, ldb, ldd, a_mn, b_mn, mode, bias=None, aux=None, accumulate=False, splits=1, max_ctas=0, ready=None):
    """Dispatches to the two-SM kernel (256 x 256 tiles on CTA pairs) for problems with enough tiles, else to the single-CTA one.
    ``ready`` (an object with flags_ptr, n, seq and wait()) marks the B operand as the target of an all-gather in flight: the
    two-SM kernel polls the peers' flags itself before its first load; the single-CTA kernel runs after ``ready.wait()``."""
    global _launches
    lib = _lib.cuda()
    _launches += 1
    tiles256 = ((M + 255) // 256) * ((N + 255) // 256)
    if mode == MODE_ACCUM:
        two_sm = TWO_SM_MIN_TILES > 0 and a_mn and b_mn and tiles256 >= 8
    else:
        two_sm = TWO_SM_MIN_TILES > 0 and not a_mn and tiles256 >= TWO_SM_MIN_TILES
    ws = cnt = None
    if two_sm:
        if mode == MODE_ACCUM:
            splits = lib.llmc_gemm2_pick_splits(M, N, K, sm_count(d.device))
            wsf, nc = ctypes.c_longlong(0), ctypes.c_int(0)
            lib.llmc_gemm2_workspace(M, N, splits, ctypes.byref(wsf), ctypes.byref(nc))
            if splits > 1:
                ws = _scratch.get("gemm_ws", wsf.value, torch.float32, d.device)
            cnt = _scratch.get("gemm2_cnt", nc.value, torch.int32, d.device, zero=True)
        if ready is not None:
            check(lib.llmc_gemm2_after_flags(_p(a), _p(b), _p(d), _p(bias), _p(aux), M, N, K, lda, ldb, ldd, int(a_mn), int(b_mn), mode,
                                             int(accumulate), splits, _p(ws), _p(cnt), ctypes.c_void_p(ready.flags_ptr), ready.n, ready.seq,
                                             _stream()), "llmc_gemm2_after_flags")
            return
        check(lib.llmc_gemm2(_p(a), _p(b), _p(d), _p(bias), _p(aux), M, N, K, lda, ldb, ldd, int(a_mn), int(b_mn), mode, int(accumulate), splits,
                             _p(ws), _p(cnt), _stream()), "llmc_gemm2")
        return
    if ready is not None:
        ready.wait()
    if mode == MODE_ACCUM and splits > 1:
        wsf, nc = ctypes.c_longlong(0), ctypes.c_int(0)
        lib.llmc_gemm_workspace(M, N, splits, ctypes.byref(wsf), ctypes.byref(nc))
        ws = _scratch.get("gemm_ws", wsf.value, torch.float32, d.device)
        cnt = _scratch.get("gemm_cnt", nc.value, torch.int32, d.device, zero=True)
    check(lib.llmc_gemm(_p(a), _p(b), _p(d), _p(bias), _p(aux), M, N, K, lda, ldb, ldd, int(a_mn), int(b_mn), mode,
                        int(accumulate), splits, _p(ws), _p(cnt), max_ctas, _stream()), "llmc_gemm")


def matmul_forward(out, inp, weight, bias=None, pre_gelu=None, ready=None):
    """out[M,OC] = inp[M,C] @ weight[OC,C]^T (+ bias).  With ``pre_gelu`` the pre-activation is stored there and
    ``out`` receives its tanh-GELU (reference: matmul_forward_cublaslt, llmc/matmul.cuh:230-242)."""
    M, C = inp.shape
    OC = weight.shape[0]
    mode = MODE_GELU if pre_gelu is not None else MODE_STORE
    gemm(inp, weight, out, M, OC, C, C, C, OC, 0, 0, mode, bias=bias, aux=pre_gelu, ready=ready)


def matmul_dgrad(dinp, dout, weight, pre_gelu=None):
    """dinp[M,C] = dout[M,OC] @ weight[OC,C]; multiplied by GELU'(pre_gelu[M,C]) if given
    (reference: matmul_backward dgrad with the DGELU epilogue, llmc/matmul.cuh:279-285)."""
    M, OC = dout.shape
    C = weight.shape[1]
    mode = MODE_DGELU if pre_gelu is not None else MODE_STORE
    gemm(dout, weight, dinp, M, C, OC, OC, C, C, 0, 1, mode, aux=pre_gelu)


def matmul_wgrad(dweight, dout, inp, accumulate=True):
    """dweight[OC,C] (+)= dout[M,OC]^T @ inp[M,C] with split-K sized to fill the SMs."""
    M, OC = dout.shape
    C = inp.shape[1]
    splits = _lib.cuda().llmc_gemm_pick_splits(OC, C, M, sm_count(dout.device))
    gemm(dout, inp, dweight, OC, C, M, OC, C, C, 1, 1, MODE_ACCUM, accumulate=accumulate, splits=splits)


def gemm_tf32(d, a, b, bias=None, accumulate=False):
    """d[M,N] (+)= a[M,K] @ b[N,K]^T (+ bias): fp32 tensors, tcgen05 kind::tf32 with fp32 accumulation (the matmul of the
    full-precision mode; the reference runs cuBLAS in TF32 there when -f 1, train_gpt2_fp32.cu / PRECISION=FP32)."""
    global _launches
    M, K = a.shape
    N = b.shape[0]
    assert a.dtype == b.dtype == d.dtype == torch.float32 and b.shape[1] == K and tuple(d.shape) == (M, N)
    assert a.stride(1) == 1 and b.stride(1) == 1 and d.stride(1) == 1
    _launches += 1
    check(_lib.cuda().llmc_gemm_tf32(_p(a), _p(b), _p(d), _p(bias), M, N, K, a.stride(0), b.stride(0), d.stride(0), int(accumulate), _stream()),
          "llmc_gemm_tf32")


def tf32_shapes_ok(*dims):
    return all(int(x) % 4 == 0 for x in dims)


def bias_grad(dbias, dout, accumulate=True):
    """dbias[OC] (+)= column sums of dout[M,OC]."""
    global _launches
    lib = _lib.cuda()
    M, OC = dout.shape
    s = _scratch.get("bias_grad", lib.llmc_bias_grad_scratch(M, OC), torch.float32, dout.device)
    _launches += 2
    check(lib.llmc_bias_grad(_p(dbias), _p(s), _p(dout), M, OC, int(accumulate), _stream()), "llmc_bias_grad")


def encoder_forward(out, tokens, wte, wpe):
    """out[B,T,C] = wte[tokens] + wpe[:T]."""
    global _launches
    B, T = tokens.shape
    C = wte.shape[1]
    _launches += 1
    check(_lib.cuda().llmc_encoder_fwd(_p(out), _p(tokens), _p(wte), _p(wpe), B, T, C, wte.shape[0], _stream()), "llmc_encoder_fwd")


def encoder_backward(dwte, dwpe, dout, tokens, accumulate_wte=True, accumulate_wpe=True, seed=0):
    """Deterministic scatter-add of dout[B,T,C] into the embedding gradients."""
    global _launches
    B, T = tokens.shape
    C = dwte.shape[1]
    V = dwte.shape[0]
    _launches += 2
    check(_lib.cuda().llmc_encoder_bwd(_p(dwte), _p(dwpe), _p(dout), _p(tokens), B, T, C, V, int(accumulate_wte),
                                       int(accumulate_wpe), seed & 0xFFFFFFFF, _stream()), "llmc_encoder_bwd")


def layernorm_forward(out, mean, rstd, inp, weight, bias):
    global _launches
    N, C = inp.shape
    _launches += 1
    check(_lib.cuda().llmc_layernorm_fwd(_p(out), _p(mean), _p(rstd), _p(inp), _p(weight), _p(bias), N, C, _stream()),
          "llmc_layernorm_fwd")


def fused_residual_forward(residual, normed, mean, rstd, inp1, inp2, weight, bias):
    """residual = inp1 + inp2; normed = LayerNorm(residual)."""
    global _launches
    N, C = inp1.shape
    _launches += 1
    check(_lib.cuda().llmc_fused_residual_fwd(_p(residual), _p(normed), _p(mean), _p(rstd), _p(inp1), _p(inp2), _p(weight),
                                              _p(bias), N, C, _stream()), "llmc_fused_residual_fwd")


def layernorm_backward(dinp, dweight, dbias, dout, inp, weight, mean, rstd, accumulate_dinp=True, accumulate_dwdb=True,
                       dcolsum=None, accumulate_dcol=True):
    """dinp (+)= dLN(dout); dweight/dbias (+)= their gradients.  ``dcolsum`` (+)= column sums of the final dinp: the bias
    gradient of the projection that wrote into the residual stream, at no extra pass over memory."""
    global _launches
    lib = _lib.cuda()
    N, C = inp.shape
    s = _scratch.get("ln_bwd", lib.llmc_layernorm_bwd_scratch(N, C), torch.float32, inp.device)
    _launches += 2
    check(lib.llmc_layernorm_bwd(_p(dinp), _p(dweight), _p(dbias), _p(s), _p(dout), _p(inp), _p(weight), _p(mean), _p(rstd),
                                 N, C, int(accumulate_dinp), int(accumulate_dwdb), _p(dcolsum), int(accumulate_dcol), _stream()),
          "llmc_layernorm_bwd")


def attention_forward(out, lse, qkv, B, T, NH):
    """out (B,T,NH,HS), lse (B,NH,T) from packed qkv (B,T,3,NH,HS); causal."""
    global _launches
    hs = qkv.numel() // (B * T * 3 * NH)
    _launches += 1
    check(_lib.cuda().llmc_attention_fwd(_p(out), _p(lse), _p(qkv), B, T, NH, hs, _stream()), "llmc_attention_fwd")


def attention_backward(dqkv, dout, qkv, out, lse, B, T, NH):
    """dqkv (B,T,3,NH,HS) from dout, the forward inputs and statistics; deterministic."""
    global _launches
    hs = qkv.numel() // (B * T * 3 * NH)
    lib = _lib.cuda()
    # row statistics and, for 64-wide heads, the per-pair dQ contributions of the single-pass kernel (csrc/attention_bwd1.cu)
    ws = _scratch.get("attn_bwd", lib.llmc_attention_bwd_workspace(B, T, NH, hs), torch.float32, qkv.device)
    _launches += 3
    check(lib.llmc_attention_bwd(_p(dqkv), _p(ws), _p(dout), _p(qkv), _p(out), _p(lse), B, T, NH, hs, _stream()),
          "llmc_attention_bwd")


def fused_classifier(logits, losses, targets, dloss, V, write_dlogits=True, accumulate_loss=False):
    """losses[n] (+)= CE(logits[n], targets[n]); logits <- dlogits * dloss in place."""
    global _launches
    N, Vp = logits.shape
    _launches += 1
    check(_lib.cuda().llmc_fused_classifier(_p(logits), _p(losses), _p(targets), float(dloss), N, V, Vp, int(write_dlogits),
                                            int(accumulate_loss), _stream()), "llmc_fused_classifier")


def gelu_forward(out, inp):
    global _launches
    _launches += 1
    check(_lib.cuda().llmc_gelu_fwd(_p(out), _p(inp), inp.numel(), _stream()), "llmc_gelu_fwd")


def gelu_backward_inplace(d_inout, inp):
    global _launches
    _launches += 1
    check(_lib.cuda().llmc_gelu_bwd_inplace(_p(d_inout), _p(inp), inp.numel(), _stream()), "llmc_gelu_bwd_inplace")


def residual_add(out, a, b):
    global _launches
    _launches += 1
    check(_lib.cuda().llmc_residual_add(_p(out), _p(a), _p(b), a.numel(), _stream()), "llmc_residual_add")


def rmsnorm_forward(out, rstd, inp, weight, eps=1e-5):
    """out = inp * rsqrt(mean(inp^2) + eps) * weight, statistics in fp32 (reference module: train_llama3.py:133-146)."""
    global _launches
    N, C = inp.shape
    _launches += 1
    check(_lib.cuda().llmc_rmsnorm_fwd(_p(out), _p(rstd), _p(inp), _p(weight), N, C, float(eps), _stream()), "llmc_rmsnorm_fwd")


def rmsnorm_fused_residual_forward(residual, normed, rstd, inp1, inp2, weight, eps=1e-5):
    """residual = inp1 + inp2; normed = RMSNorm(residual)."""
    global _launches
    N, C = inp1.shape
    _launches += 1
    check(_lib.cuda().llmc_rmsnorm_fused_residual_fwd(_p(residual), _p(normed), _p(rstd), _p(inp1), _p(inp2), _p(weight), N, C,
                                                      float(eps), _stream()), "llmc_rmsnorm_fused_residual_fwd")


def rmsnorm_backward(dinp, dweight, dout, inp, weight, rstd, accumulate_dinp=True, accumulate_dw=True):
    """dinp (+)= dRMSNorm(dout); dweight (+)= its gradient."""
    global _launches
    lib = _lib.cuda()
    N, C = inp.shape
    s = _scratch.get("rms_bwd", lib.llmc_rmsnorm_bwd_scratch(N, C), torch.float32, inp.device)
    _launches += 2
    check(lib.llmc_rmsnorm_bwd(_p(dinp), _p(dweight), _p(s), _p(dout), _p(inp), _p(weight), _p(rstd), N, C, int(accumulate_dinp),
                               int(accumulate_dw), _stream()), "llmc_rmsnorm_bwd")


def rope_forward(packed, raw, freqs, T, NH, NKV):
    """raw (N, (NH + 2 NKV) * HS) -> packed (N, 3, NH, HS): rotary embedding on queries and keys, key / value heads repeated
    NH / NKV times (reference: apply_rotary_emb + repeat_kv, train_llama3.py:107-117 and :59-68).  freqs: (maxT, HS/2, 2) fp32."""
    global _launches
    N = raw.shape[0]
    HS = raw.shape[1] // (NH + 2 * NKV)
    _launches += 1
    check(_lib.cuda().llmc_rope_fwd(_p(packed), _p(raw), _p(freqs), N, T, NH, NKV, HS, _stream()), "llmc_rope_fwd")


def rope_backward(draw, dpacked, freqs, T, NH, NKV):
    """Gradient of ``rope_forward``: inverse rotation, gradients of repeated heads summed over their group."""
    global _launches
    N = draw.shape[0]
    HS = draw.shape[1] // (NH + 2 * NKV)
    _launches += 1
    check(_lib.cuda().llmc_rope_bwd(_p(draw), _p(dpacked), _p(freqs), N, T, NH, NKV, HS, _stream()), "llmc_rope_bwd")


def swiglu_forward(h, x12):
    """h = x12[:, :H] * silu(x12[:, H:])."""
    global _launches
    N, H = h.shape
    _launches += 1
    check(_lib.cuda().llmc_swiglu_fwd(_p(h), _p(x12), N, H, _stream()), "llmc_swiglu_fwd")


def swiglu_backward(dx12, dh, x12):
    """dx12 = gradient of ``swiglu_forward`` with respect to both halves of x12."""
    global _launches
    N, H = dh.shape
    _launches += 1
    check(_lib.cuda().llmc_swiglu_bwd(_p(dx12), _p(dh), _p(x12), N, H, _stream()), "llmc_swiglu_bwd")


def rope_cache(q, kcache, vcache, raw, freqs, Tq, start_pos, NH, NKV, pos=None):
    """Rotary embedding of the Tq new tokens per batch row at positions start_pos.., queries to ``q`` (N, NH, HS), rotated keys
    and the values into their slots of the caches (B, Tmax, NKV, HS) (reference: CausalSelfAttention.forward with
    ``use_kv``, train_llama3.py:167-180).  ``pos`` (a one-element int32 device tensor) replaces start_pos at run time, for
    steps that are replayed from a CUDA graph."""
    global _launches
    N = raw.shape[0]
    HS = raw.shape[1] // (NH + 2 * NKV)
    _launches += 1
    check(_lib.cuda().llmc_rope_cache(_p(q), _p(kcache), _p(vcache), _p(raw), _p(freqs), freqs.shape[0], N // Tq, Tq, kcache.shape[1],
                                      start_pos, NH, NKV, HS, _p(pos), _stream()), "llmc_rope_cache")


def cached_attention(out, q, kcache, vcache, Tq, start_pos, NH, NKV, pos=None):
    """out (N, NH, HS): causal attention of the Tq new queries per batch row over cache positions 0 .. start_pos + t."""
    global _launches
    lib = _lib.cuda()
    N = q.shape[0]
    HS = kcache.shape[-1]
    B, Tmax = N // Tq, kcache.shape[1]
    # decoding steps (few query rows per cached head, head width 64 or 128) take the split-key kernel and its workspace; the
    # buffer is kept per device, so a step captured in a CUDA graph replays on the same addresses
    words = lib.llmc_cached_attention_workspace(B, Tq, Tmax, NH, NKV, HS)
    ws = _scratch.get("cached_attention", words, torch.float32, q.device) if words > 0 else None
    _launches += 2 if words > 0 else 1
    check(lib.llmc_cached_attention(_p(out), _p(q), _p(kcache), _p(vcache), B, Tq, Tmax, start_pos, NH, NKV, HS, _p(pos), _p(ws), _stream()),
          "llmc_cached_attention")


def matmul_skinny(out, inp, weight):
    """out[M,OC] = inp[M,C] @ weight[OC,C]^T for at most 8 rows: the weight-streaming kernel of decoding steps (csrc/decode.cu)."""
    global _launches
    M, C = inp.shape
    OC = weight.shape[0]
    _launches += 1
    check(_lib.cuda().llmc_skinny_gemm(_p(out), _p(inp), _p(weight), M, OC, C, inp.stride(0), weight.stride(0), out.stride(0), _stream()),
          "llmc_skinny_gemm")


def make_table(views):
    """views: list of dicts(p_base, p_stride, o_base, o_stride, n, L, wd, seed[, l_base])."""
    tab = TensorTable()
    assert len(views) <= 16
    for i, v in enumerate(views):
        t = tab.t[i]
        t.p_base, t.p_stride, t.o_base, t.o_stride = v["p_base"], v["p_stride"], v["o_base"], v["o_stride"]
        t.n, t.L, t.wd, t.seed = v["n"], v["L"], float(v.get("wd", 0.0)), int(v.get("seed", 0)) & 0xFFFFFFFF
        t.pad = int(v.get("l_base", 0))        # layer index of the view's first slice (enters the stochastic-rounding noise index)
    tab.count = len(views)
    return tab


def global_norm_sq(out, grads, views):
    """out[0] = sum of squares of the gradient elements described by ``views`` (deterministic)."""
    global _launches
    lib = _lib.cuda()
    part = _scratch.get("norm_sq", lib.llmc_norm_sq_scratch(), torch.float32, grads.device)
    tab = make_table(views)
    _launches += 2
    check(lib.llmc_global_norm_sq(_p(out), _p(part), _p(grads), ctypes.byref(tab), _stream()), "llmc_global_norm_sq")


def sum_scaled(out, terms, scale=1.0):
    """out[0] = scale * sum(terms) over fp32 device tensors, one block, fixed summation tree (the mean loss of a step)."""
    global _launches
    _launches += 1
    check(_lib.cuda().llmc_sum_f32(_p(out), _p(terms), terms.numel(), float(scale), _stream()), "llmc_sum_f32")


def adamw_update(params, master, grads, m, v, views, lr, beta1, beta2, eps, t, grad_scale=1.0, norm_sq=None, grad_clip=1.0):
    """AdamW on the views; bf16 params are stochastically rounded from the fp32 result."""
    global _launches
    tab = make_table(views)
    _launches += 1
    check(_lib.cuda().llmc_adamw(_p(params), _p(master), _p(grads), _p(m), _p(v), ctypes.byref(tab), lr, beta1, beta2, eps,
                                 int(t), grad_scale, _p(norm_sq), grad_clip, _stream()), "llmc_adamw")


def params_from_master(params, master, views):
    global _launches
    tab = make_table(views)
    _launches += 1
    check(_lib.cuda().llmc_params_from_master(_p(params), _p(master), ctypes.byref(tab), _stream()), "llmc_params_from_master")


def master_from_params(master, params, views):
    global _launches
    tab = make_table(views)
    _launches += 1
    check(_lib.cuda().llmc_master_from_params(_p(master), _p(params), ctypes.byref(tab), _stream()), "llmc_master_from_params")
