"""Launchers of the full-precision (fp32) kernels of csrc/fp32_ops.cu: the GPT-2 operator set for fp32 tensors on a CUDA device
(the trainer's ``-dt fp32`` mode; reference: the kernels of train_gpt2_fp32.cu).  Signatures match ``kernels`` and ``reference``:
outputs are written in place.  The matmuls of this mode stay where they were (``reference.matmul_*``: this library's TF32
tensor-core kernel with ``-f 1``, cuBLAS in IEEE fp32 otherwise); the two batched products of the attention block run on
cuBLAS through ``torch.bmm``, as the reference's legacy trainer does, around this library's permutation and softmax kernels.
"""
import ctypes
import math

import torch

from .. import _lib
from .._lib import check
from . import kernels
from .kernels import _p, _scratch, _stream
from .reference import matmul_dgrad, matmul_forward, matmul_wgrad     # noqa: F401  (re-exported: the matmuls of this mode, see above)

F32 = torch.float32


def _lib_():
    return _lib.cuda()


def _c(*tensors):
    for t in tensors:
        if t is not None:
            assert t.is_cuda and t.dtype == F32 and t.is_contiguous(), "fp32 kernels want contiguous fp32 device tensors"


def _count(n=1):
    kernels._launches += n


def gelu_forward(out, inp):
    _c(out, inp); _count()
    check(_lib_().llmc_f32_gelu_fwd(_p(out), _p(inp), inp.numel(), _stream()), "llmc_f32_gelu_fwd")


def gelu_backward_inplace(d_inout, inp):
    _c(d_inout, inp); _count()
    check(_lib_().llmc_f32_gelu_bwd(_p(d_inout), _p(inp), inp.numel(), _stream()), "llmc_f32_gelu_bwd")


def residual_add(out, a, b):
    _c(out, a, b); _count()
    check(_lib_().llmc_f32_residual_add(_p(out), _p(a), _p(b), out.numel(), _stream()), "llmc_f32_residual_add")


def encoder_forward(out, tokens, wte, wpe):
    B, T = tokens.shape
    C = wte.shape[1]
    _c(out, wte, wpe); _count()
    check(_lib_().llmc_f32_encoder_fwd(_p(out), _p(tokens), _p(wte), _p(wpe), B, T, C, wte.shape[0], _stream()), "llmc_f32_encoder_fwd")


def encoder_backward(dwte, dwpe, dout, tokens, accumulate_wte=True, accumulate_wpe=True, seed=0):
    B, T = tokens.shape
    C = dwte.shape[1]
    _c(dwte, dwpe, dout); _count(2)
    check(_lib_().llmc_f32_encoder_bwd(_p(dwte), _p(dwpe), _p(dout), _p(tokens), B, T, C, dwte.shape[0], int(accumulate_wte),
                                       int(accumulate_wpe), _stream()), "llmc_f32_encoder_bwd")


def layernorm_forward(out, mean, rstd, inp, weight, bias):
    C = inp.shape[-1]
    rows = inp.numel() // C
    _c(out, mean, rstd, inp, weight, bias); _count()
    check(_lib_().llmc_f32_layernorm_fwd(_p(out), _p(mean), _p(rstd), None, _p(inp), None, _p(weight), _p(bias), rows, C, _stream()),
          "llmc_f32_layernorm_fwd")


def fused_residual_forward(residual, normed, mean, rstd, inp1, inp2, weight, bias):
    C = inp1.shape[-1]
    rows = inp1.numel() // C
    _c(residual, normed, mean, rstd, inp1, inp2, weight, bias); _count()
    check(_lib_().llmc_f32_layernorm_fwd(_p(normed), _p(mean), _p(rstd), _p(residual), _p(inp1), _p(inp2), _p(weight), _p(bias), rows, C,
                                         _stream()), "llmc_f32_layernorm_fwd")


def layernorm_backward(dinp, dweight, dbias, dout, inp, weight, mean, rstd, accumulate_dinp=True, accumulate_dwdb=True,
                       dcolsum=None, accumulate_dcol=True):
    lib = _lib_()
    C = inp.shape[-1]
    rows = inp.numel() // C
    _c(dinp, dweight, dbias, dout, inp, weight, mean, rstd, dcolsum); _count(2)
    s = _scratch.get("f32_ln_bwd", lib.llmc_f32_layernorm_bwd_scratch(rows, C), F32, inp.device)
    check(lib.llmc_f32_layernorm_bwd(_p(dinp), _p(dweight), _p(dbias), _p(dcolsum), _p(s), _p(dout), _p(inp), _p(weight), _p(mean),
                                     _p(rstd), rows, C, int(accumulate_dinp), int(accumulate_dwdb), int(accumulate_dcol), _stream()),
          "llmc_f32_layernorm_bwd")


def bias_grad(dbias, dout, accumulate=True):
    lib = _lib_()
    M, OC = dout.shape
    _c(dbias, dout); _count(2)
    s = _scratch.get("f32_bias_grad", lib.llmc_f32_bias_grad_scratch(M, OC), F32, dout.device)
    check(lib.llmc_f32_bias_grad(_p(dbias), _p(s), _p(dout), M, OC, int(accumulate), _stream()), "llmc_f32_bias_grad")


def fused_classifier(logits, losses, targets, dloss, V, write_dlogits=True, accumulate_loss=False):
    N, Vp = logits.shape
    _c(logits, losses); _count()
    check(_lib_().llmc_f32_classifier(_p(logits), _p(losses), _p(targets), float(dloss), N, V, Vp, int(write_dlogits),
                                      int(accumulate_loss), _stream()), "llmc_f32_classifier")


def _attention_buffers(B, T, NH, hs, device, backward):
    sep = _scratch.get("f32_att_sep", 3 * B * NH * T * hs, F32, device)[:3 * B * NH * T * hs].view(3, B * NH, T, hs)
    att = _scratch.get("f32_att", B * NH * T * T, F32, device)[:B * NH * T * T].view(B * NH, T, T)
    y = _scratch.get("f32_att_y", B * NH * T * hs, F32, device)[:B * NH * T * hs].view(B * NH, T, hs)
    if not backward:
        return sep, att, y
    datt = _scratch.get("f32_datt", B * NH * T * T, F32, device)[:B * NH * T * T].view(B * NH, T, T)
    dsep = _scratch.get("f32_att_dsep", 3 * B * NH * T * hs, F32, device)[:3 * B * NH * T * hs].view(3, B * NH, T, hs)
    return sep, att, y, datt, dsep


def attention_forward(out, lse, qkv, B, T, NH):
    """out (B,T,NH*hs) = causal attention of the packed qkv (B,T,3,NH,hs); lse (B,NH,T) = log-sum-exp of the scaled scores."""
    lib = _lib_()
    hs = qkv.numel() // (B * T * 3 * NH)
    _c(out, lse, qkv); _count(3)
    sep, att, y = _attention_buffers(B, T, NH, hs, qkv.device, False)
    check(lib.llmc_f32_permute_qkv(_p(sep), _p(qkv), B, T, NH, hs, 1, _stream()), "llmc_f32_permute_qkv")
    torch.bmm(sep[0], sep[1].transpose(1, 2), out=att)
    check(lib.llmc_f32_softmax_causal(_p(att), _p(lse), None, 1.0 / math.sqrt(hs), B * NH * T, T, _stream()), "llmc_f32_softmax_causal")
    torch.bmm(att, sep[2], out=y)
    check(lib.llmc_f32_permute_heads(_p(y), _p(out), B, T, NH, hs, 1, _stream()), "llmc_f32_permute_heads")


def attention_backward(dqkv, dout, qkv, out, lse, B, T, NH):
    """dqkv (B,T,3,NH,hs) from dout (B,T,NH*hs); the probabilities are recomputed from qkv and the stored lse."""
    lib = _lib_()
    hs = qkv.numel() // (B * T * 3 * NH)
    scale = 1.0 / math.sqrt(hs)
    _c(dqkv, dout, qkv, lse); _count(5)
    sep, att, dy, datt, dsep = _attention_buffers(B, T, NH, hs, qkv.device, True)
    check(lib.llmc_f32_permute_qkv(_p(sep), _p(qkv), B, T, NH, hs, 1, _stream()), "llmc_f32_permute_qkv")
    torch.bmm(sep[0], sep[1].transpose(1, 2), out=att)
    check(lib.llmc_f32_softmax_causal(_p(att), None, _p(lse), scale, B * NH * T, T, _stream()), "llmc_f32_softmax_causal")
    check(lib.llmc_f32_permute_heads(_p(dy), _p(dout), B, T, NH, hs, 0, _stream()), "llmc_f32_permute_heads")
    torch.bmm(att.transpose(1, 2), dy, out=dsep[2])                       # dV = P^T dO
    torch.bmm(dy, sep[2].transpose(1, 2), out=datt)                       # dP = dO V^T
    check(lib.llmc_f32_softmax_causal_bwd(_p(datt), _p(att), scale, B * NH * T, T, _stream()), "llmc_f32_softmax_causal_bwd")
    torch.bmm(datt, sep[1], out=dsep[0])                                  # dQ = dS K
    torch.bmm(datt.transpose(1, 2), sep[0], out=dsep[1])                  # dK = dS^T Q
    check(lib.llmc_f32_permute_qkv(_p(dsep), _p(dqkv), B, T, NH, hs, 0, _stream()), "llmc_f32_permute_qkv")


def global_norm_sq(out, grads, views):
    """out[0] = sum of squares of the listed slices of ``grads``, added in a fixed order."""
    lib = _lib_()
    _c(grads)
    per = lib.llmc_f32_sumsq_partials_per_slice()
    total = sum(v["L"] for v in views) * per
    part = _scratch.get("f32_sumsq", total, F32, grads.device)
    off = 0
    for v in views:
        _count()
        check(lib.llmc_f32_sumsq(ctypes.c_void_p(part.data_ptr() + 4 * off), _p(grads), v["p_base"], v["p_stride"], v["n"], v["L"], _stream()),
              "llmc_f32_sumsq")
        off += v["L"] * per
    _count()
    check(lib.llmc_sum_f32(_p(out), _p(part), total, 1.0, _stream()), "llmc_sum_f32")


def adamw_update(params, master, grads, m, v, views, lr, beta1, beta2, eps, t, grad_scale=1.0, norm_sq=None, grad_clip=1.0):
    """AdamW on fp32 parameters (round to nearest; no stochastic rounding is needed).  The clip coefficient is computed on the
    device from ``norm_sq``; a non-finite norm leaves parameters and state untouched."""
    lib = _lib_()
    _c(params, master, grads, m, v)
    for tv in views:
        _count()
        check(lib.llmc_f32_adamw(_p(params), _p(master), _p(grads), _p(m), _p(v), tv["p_base"], tv["p_stride"], tv["o_base"], tv["o_stride"],
                                 tv["n"], tv["L"], float(lr), float(beta1), float(beta2), int(t), float(eps), float(tv.get("wd", 0.0)),
                                 float(grad_scale), _p(norm_sq), float(grad_clip), _stream()), "llmc_f32_adamw")


def params_from_master(params, master, views):
    lib = _lib_()
    _c(params, master)
    for tv in views:
        _count()
        check(lib.llmc_f32_copy_slices(_p(params), _p(master), tv["p_base"], tv["p_stride"], tv["o_base"], tv["o_stride"], tv["n"], tv["L"],
                                       _stream()), "llmc_f32_copy_slices")


def master_from_params(master, params, views):
    lib = _lib_()
    _c(params, master)
    for tv in views:
        _count()
        check(lib.llmc_f32_copy_slices(_p(master), _p(params), tv["o_base"], tv["o_stride"], tv["p_base"], tv["p_stride"], tv["n"], tv["L"],
                                       _stream()), "llmc_f32_copy_slices")
