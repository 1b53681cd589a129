"""Plain PyTorch restatement of every operator (fp32 math, any storage dtype).

It is the CPU execution path of the framework (fp32 training on the host, the counterpart of the
reference's train_gpt2.c), the numerics oracle the kernel tests compare against, and the fp32 mode on a GPU
(``-dt fp32`` on a CUDA device, the counterpart of the reference's legacy train_gpt2_fp32.cu: every tensor fp32, the
operators executed by PyTorch's own CUDA library on the tensors' device).  Signatures match ``kernels`` exactly:
outputs are written in place.
"""
import math

import torch

GELU_K = math.sqrt(2.0 / math.pi)


def _f(t):
    return t.float()


def gelu(x):
    return 0.5 * x * (1.0 + torch.tanh(GELU_K * (x + 0.044715 * x ** 3)))


def gelu_grad(x):
    t = torch.tanh(GELU_K * (x + 0.044715 * x ** 3))
    return 0.5 * (1.0 + t) + x * 0.5 * (1.0 - t * t) * GELU_K * (1.0 + 3.0 * 0.044715 * x * x)


def _tf32_kernel(*tensors):
    """True if the product should run on this library's TF32 tensor-core kernel: fp32 tensors on a CUDA device with TF32 allowed
    (the -f switch of the trainer).  Otherwise the product is PyTorch's."""
    t0 = tensors[0]
    return (t0.is_cuda and torch.backends.cuda.matmul.allow_tf32 and all(t.dtype == torch.float32 and t.dim() == 2 for t in tensors)
            and all(x % 4 == 0 for t in tensors for x in t.shape))


def matmul_forward(out, inp, weight, bias=None, pre_gelu=None, ready=None):
    if ready is not None:
        ready.wait()
    if _tf32_kernel(out, inp, weight):
        from . import kernels
        dst = pre_gelu if pre_gelu is not None else out
        kernels.gemm_tf32(dst, inp, weight, bias)
        if pre_gelu is not None:
            out.copy_(gelu(pre_gelu))
        return
    y = _f(inp) @ _f(weight).t()
    if bias is not None:
        y = y + _f(bias)
    if pre_gelu is not None:
        pre_gelu.copy_(y)
        y = gelu(_f(pre_gelu))
    out.copy_(y)


def matmul_dgrad(dinp, dout, weight, pre_gelu=None):
    if _tf32_kernel(dinp, dout, weight):
        from . import kernels
        kernels.gemm_tf32(dinp, dout, weight.t().contiguous())        # the kernel wants both operands K-major
        if pre_gelu is not None:
            dinp.mul_(gelu_grad(pre_gelu))
        return
    y = _f(dout) @ _f(weight)
    if pre_gelu is not None:
        y = y * gelu_grad(_f(pre_gelu))
    dinp.copy_(y)


def matmul_wgrad(dweight, dout, inp, accumulate=True):
    if _tf32_kernel(dweight, dout, inp):
        from . import kernels
        kernels.gemm_tf32(dweight, dout.t().contiguous(), inp.t().contiguous(), None, accumulate)
        return
    y = _f(dout).t() @ _f(inp)
    if accumulate:
        y = y + _f(dweight)
    dweight.copy_(y)


def bias_grad(dbias, dout, accumulate=True):
    y = _f(dout).sum(0)
    if accumulate:
        y = y + _f(dbias)
    dbias.copy_(y)


def encoder_forward(out, tokens, wte, wpe):
    B, T = tokens.shape
    x = _f(wte)[tokens.long()]
    if wpe is not None:
        x = x + _f(wpe)[:T].unsqueeze(0)
    out.copy_(x.view_as(out))


def encoder_backward(dwte, dwpe, dout, tokens, accumulate_wte=True, accumulate_wpe=True, seed=0):
    B, T = tokens.shape
    C = dwte.shape[1]
    d = _f(dout).view(B, T, C)
    if dwpe is not None:
        gp = d.sum(0)
        if accumulate_wpe:
            gp = gp + _f(dwpe[:T])
        dwpe[:T].copy_(gp)
    gw = torch.zeros(dwte.shape, dtype=torch.float32, device=dwte.device)
    gw.index_add_(0, tokens.reshape(-1).long(), d.reshape(B * T, C))
    if accumulate_wte:
        gw = gw + _f(dwte)
    dwte.copy_(gw)


def _ln(x, weight, bias):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    rstd = torch.rsqrt(var + 1e-5)
    return (x - mean) * rstd * _f(weight) + _f(bias), mean.squeeze(-1), rstd.squeeze(-1)


def layernorm_forward(out, mean, rstd, inp, weight, bias):
    y, m, r = _ln(_f(inp), weight, bias)
    out.copy_(y)
    if mean is not None:
        mean.copy_(m)
    if rstd is not None:
        rstd.copy_(r)


def fused_residual_forward(residual, normed, mean, rstd, inp1, inp2, weight, bias):
    residual.copy_(_f(inp1) + _f(inp2))
    layernorm_forward(normed, mean, rstd, residual, weight, bias)


def layernorm_backward(dinp, dweight, dbias, dout, inp, weight, mean, rstd, accumulate_dinp=True, accumulate_dwdb=True,
                       dcolsum=None, accumulate_dcol=True):
    dy, x, w = _f(dout), _f(inp), _f(weight)
    norm = (x - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)
    dnorm = dy * w
    dx = (dnorm - dnorm.mean(-1, keepdim=True) - norm * (dnorm * norm).mean(-1, keepdim=True)) * rstd.unsqueeze(-1)
    dw = (dy * norm).sum(0)
    db = dy.sum(0)
    if accumulate_dinp:
        dx = dx + _f(dinp)
    if accumulate_dwdb:
        dw, db = dw + _f(dweight), db + _f(dbias)
    dinp.copy_(dx)
    dweight.copy_(dw)
    dbias.copy_(db)
    if dcolsum is not None:
        cs = _f(dinp).sum(0)
        if accumulate_dcol:
            cs = cs + _f(dcolsum)
        dcolsum.copy_(cs)


def _split_qkv(qkv, B, T, NH):
    hs = qkv.numel() // (B * T * 3 * NH)
    x = _f(qkv).view(B, T, 3, NH, hs)
    return x[:, :, 0].transpose(1, 2), x[:, :, 1].transpose(1, 2), x[:, :, 2].transpose(1, 2), hs   # (B,NH,T,hs)


def attention_forward(out, lse, qkv, B, T, NH):
    q, k, v, hs = _split_qkv(qkv, B, T, NH)
    att = (q @ k.transpose(-1, -2)) / math.sqrt(hs)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    att = att.masked_fill(~mask, float("-inf"))
    lse.copy_(torch.logsumexp(att, -1).view_as(lse))
    y = torch.softmax(att, -1) @ v
    out.copy_(y.transpose(1, 2).reshape(out.shape))


def attention_backward(dqkv, dout, qkv, out, lse, B, T, NH):
    q, k, v, hs = _split_qkv(qkv, B, T, NH)
    scale = 1.0 / math.sqrt(hs)
    att = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    p = torch.exp(att - _f(lse).view(B, NH, T, 1)).masked_fill(~mask, 0.0)
    do = _f(dout).view(B, T, NH, hs).transpose(1, 2)
    o = _f(out).view(B, T, NH, hs).transpose(1, 2)
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    delta = (do * o).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    res = torch.stack([dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)], dim=2)   # (B,T,3,NH,hs)
    dqkv.copy_(res.reshape(dqkv.shape))


def fused_classifier(logits, losses, targets, dloss, V, write_dlogits=True, accumulate_loss=False):
    N, Vp = logits.shape
    x = _f(logits)[:, :V]
    lp = torch.log_softmax(x, -1)
    loss = -lp.gather(1, targets.long().view(-1, 1)).squeeze(1)
    if accumulate_loss:
        loss = loss + losses
    losses.copy_(loss)
    if write_dlogits:
        g = torch.exp(lp)
        g.scatter_add_(1, targets.long().view(-1, 1), -torch.ones(N, 1, device=logits.device))
        full = torch.zeros(N, Vp, device=logits.device)
        full[:, :V] = g * dloss
        logits.copy_(full)


def gelu_forward(out, inp):
    out.copy_(gelu(_f(inp)))


def gelu_backward_inplace(d_inout, inp):
    d_inout.copy_(_f(d_inout) * gelu_grad(_f(inp)))


def residual_add(out, a, b):
    out.copy_(_f(a) + _f(b))


def _view_slices(v):
    for l in range(v["L"]):
        yield (v["p_base"] + l * v["p_stride"], v["o_base"] + l * v["o_stride"], v["n"])


def global_norm_sq(out, grads, views):
    acc = torch.zeros((), dtype=torch.float32, device=grads.device)
    for v in views:
        for pb, _, n in _view_slices(v):
            acc = acc + (_f(grads[pb:pb + n]) ** 2).sum()
    out[0] = acc


def sum_scaled(out, terms, scale=1.0):
    out[0] = terms.sum() * scale


def adamw_update(params, master, grads, m, v, views, lr, beta1, beta2, eps, t, grad_scale=1.0, norm_sq=None, grad_clip=1.0):
    """Round-to-nearest instead of stochastic rounding (the CPU path keeps fp32 parameters anyway)."""
    scale = grad_scale
    if norm_sq is not None:
        nsq = float(norm_sq[0])
        if not math.isfinite(nsq):
            return
        nrm = math.sqrt(nsq)
        if nrm > grad_clip:
            scale = grad_scale * grad_clip / nrm
    bc1, bc2 = 1.0 - beta1 ** t, 1.0 - beta2 ** t
    for tv in views:
        for pb, ob, n in _view_slices(tv):
            g = _f(grads[pb:pb + n]) * scale
            mm = m[ob:ob + n]
            vv = v[ob:ob + n]
            mm.mul_(beta1).add_(g, alpha=1.0 - beta1)
            vv.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
            old = master[ob:ob + n] if master is not None else _f(params[pb:pb + n])
            new = old - lr * ((mm / bc1) / (torch.sqrt(vv / bc2) + eps) + tv.get("wd", 0.0) * old)
            params[pb:pb + n].copy_(new)
            if master is not None:
                master[ob:ob + n].copy_(new)


def params_from_master(params, master, views):
    for tv in views:
        for pb, ob, n in _view_slices(tv):
            params[pb:pb + n].copy_(master[ob:ob + n])


def master_from_params(master, params, views):
    for tv in views:
        for pb, ob, n in _view_slices(tv):
            master[ob:ob + n].copy_(_f(params[pb:pb + n]))


# ---------------------------------------------------------------------------------------------------------------
# LLaMA-3 family operators

def rmsnorm_forward(out, rstd, inp, weight, eps=1e-5):
    x = _f(inp)
    rs = torch.rsqrt(x.pow(2).mean(-1) + eps)
    n = (x * rs.unsqueeze(-1)).to(out.dtype)          # rounded to the activation type before the weight is applied
    out.copy_(_f(n) * _f(weight))
    if rstd is not None:
        rstd.copy_(rs)


def rmsnorm_fused_residual_forward(residual, normed, rstd, inp1, inp2, weight, eps=1e-5):
    residual.copy_(_f(inp1) + _f(inp2))
    rmsnorm_forward(normed, rstd, residual, weight, eps)


def rmsnorm_backward(dinp, dweight, dout, inp, weight, rstd, accumulate_dinp=True, accumulate_dw=True):
    x, dy, w, rs = _f(inp), _f(dout), _f(weight), _f(rstd).unsqueeze(-1)
    n = x * rs
    dn = dy * w
    dx = (dn - n * (dn * n).mean(-1, keepdim=True)) * rs
    dw = (dy * n).sum(0)
    if accumulate_dinp:
        dx = dx + _f(dinp)
    if accumulate_dw:
        dw = dw + _f(dweight)
    dinp.copy_(dx)
    dweight.copy_(dw)


def _rotate(x, freqs, T, sign):
    """x (N, heads, HS) rotated pairwise by the angles of freqs (maxT, HS/2, 2) at position n % T."""
    N, heads, HS = x.shape
    f = _f(freqs)[:T].repeat(N // T, 1, 1)                      # (N, HS/2, 2)
    c, s = f[..., 0].unsqueeze(1), f[..., 1].unsqueeze(1) * sign
    re, im = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = re * c - im * s
    out[..., 1::2] = re * s + im * c
    return out


def rope_forward(packed, raw, freqs, T, NH, NKV):
    N = raw.shape[0]
    HS = raw.shape[1] // (NH + 2 * NKV)
    rep = NH // NKV
    x = _f(raw).view(N, NH + 2 * NKV, HS)
    q = _rotate(x[:, :NH], freqs, T, 1.0).to(packed.dtype)
    k = _rotate(x[:, NH:NH + NKV], freqs, T, 1.0).to(packed.dtype)
    v = x[:, NH + NKV:].to(packed.dtype)
    out = packed.view(N, 3, NH, HS)
    out[:, 0].copy_(q)
    out[:, 1].copy_(k.repeat_interleave(rep, dim=1))
    out[:, 2].copy_(v.repeat_interleave(rep, dim=1))


def rope_backward(draw, dpacked, freqs, T, NH, NKV):
    N = draw.shape[0]
    HS = draw.shape[1] // (NH + 2 * NKV)
    rep = NH // NKV
    d = _f(dpacked).view(N, 3, NH, HS)
    dq = _rotate(d[:, 0], freqs, T, -1.0)
    dk = _rotate(d[:, 1].reshape(N, NKV, rep, HS).sum(2), freqs, T, -1.0)
    dv = d[:, 2].reshape(N, NKV, rep, HS).sum(2)
    draw.copy_(torch.cat([dq, dk, dv], dim=1).view(N, -1))


def rope_cache(q, kcache, vcache, raw, freqs, Tq, start_pos, NH, NKV, pos=None):
    if pos is not None:
        start_pos = int(pos.item())
    N = raw.shape[0]
    B = N // Tq
    HS = raw.shape[1] // (NH + 2 * NKV)
    x = _f(raw).view(N, NH + 2 * NKV, HS)
    f = freqs[start_pos:start_pos + Tq]
    q.view(N, NH, HS).copy_(_rotate(x[:, :NH], f, Tq, 1.0))
    kcache[:B, start_pos:start_pos + Tq].copy_(_rotate(x[:, NH:NH + NKV], f, Tq, 1.0).view(B, Tq, NKV, HS))
    vcache[:B, start_pos:start_pos + Tq].copy_(x[:, NH + NKV:].view(B, Tq, NKV, HS))


def cached_attention(out, q, kcache, vcache, Tq, start_pos, NH, NKV, pos=None):
    if pos is not None:
        start_pos = int(pos.item())
    N = q.shape[0]
    B = N // Tq
    HS = kcache.shape[-1]
    rep = NH // NKV
    S = start_pos + Tq
    qq = _f(q).view(B, Tq, NH, HS).transpose(1, 2)                                    # (B, NH, Tq, HS)
    k = _f(kcache[:B, :S]).repeat_interleave(rep, dim=2).transpose(1, 2)              # (B, NH, S, HS)
    v = _f(vcache[:B, :S]).repeat_interleave(rep, dim=2).transpose(1, 2)
    att = qq @ k.transpose(-1, -2) / math.sqrt(HS)
    key = torch.arange(S, device=att.device).view(1, S)
    qry = torch.arange(Tq, device=att.device).view(Tq, 1) + start_pos
    att = att.masked_fill(key > qry, float("-inf"))
    y = torch.softmax(att, dim=-1) @ v                                                # (B, NH, Tq, HS)
    out.view(B, Tq, NH, HS).copy_(y.transpose(1, 2))


def matmul_skinny(out, inp, weight):
    out.copy_(_f(inp) @ _f(weight).t())


def swiglu_forward(h, x12):
    H = h.shape[1]
    x = _f(x12)
    h.copy_(x[:, :H] * torch.nn.functional.silu(x[:, H:]))


def swiglu_backward(dx12, dh, x12):
    H = dh.shape[1]
    x, dy = _f(x12), _f(dh)
    x1, x2 = x[:, :H], x[:, H:]
    sg = torch.sigmoid(x2)
    dx12[:, :H].copy_(dy * x2 * sg)
    dx12[:, H:].copy_(dy * x1 * sg * (1.0 + x2 * (1.0 - sg)))
