"""Numerics of every sm_100a kernel against the plain PyTorch fp32 restatement of the same operator
(the scheme of the reference's dev/cuda/*.cu files: CPU reference -> validate_result)."""
import math

import pytest
import torch

from llmc_b200.ops import kernels as KN
from llmc_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, scale=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, atol, rtol, what):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, "%s: %d/%d elements off, max err %.4g (max ref %.4g)" % (what, bad, err.numel(), err.max().item(), want.abs().max().item())


GEMM_SHAPES = [(256, 256, 64), (128, 512, 256), (384, 768, 768), (200, 264, 136), (1024, 2304, 768), (512, 1600, 1600)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_matmul_forward_bias(M, N, K):
    inp, w, b = rnd(M, K), rnd(N, K, scale=0.05), rnd(N)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.matmul_forward(out, inp.to(DEV), w.to(DEV), b.to(DEV))
    ref = torch.empty(M, N)
    R.matmul_forward(ref, inp, w, b)
    close(out, ref, 2e-2, 1e-2, "matmul_forward")


def test_matmul_forward_nobias_canary():
    M, N, K_ = 300, 520, 320
    inp, w = rnd(M, K_), rnd(N, K_, scale=0.05)
    # canary rows after the output must stay untouched
    buf = torch.full((M + 8, N), 7.0, dtype=torch.bfloat16, device=DEV)
    KN.matmul_forward(buf[:M], inp.to(DEV), w.to(DEV), None)
    ref = torch.empty(M, N)
    R.matmul_forward(ref, inp, w, None)
    close(buf[:M], ref, 2e-2, 1e-2, "matmul_forward nobias")
    assert (buf[M:] == 7.0).all()


@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (1024, 3072, 768)])
def test_matmul_forward_gelu(M, N, K):
    inp, w, b = rnd(M, K), rnd(N, K, scale=0.05), rnd(N)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    pre = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    KN.matmul_forward(out, inp.to(DEV), w.to(DEV), b.to(DEV), pre_gelu=pre)
    ref, refpre = torch.empty(M, N), torch.empty(M, N)
    R.matmul_forward(ref, inp, w, b, pre_gelu=refpre)
    close(pre, refpre, 2e-2, 1e-2, "pre_gelu")
    close(out, ref, 2e-2, 1e-2, "gelu out")


@pytest.mark.parametrize("M,OC,C", [(256, 256, 128), (384, 3072, 768), (200, 264, 136), (512, 1600, 6400)])
def test_matmul_dgrad(M, OC, C):
    dout, w = rnd(M, OC), rnd(OC, C, scale=0.05)
    dinp = torch.empty(M, C, dtype=torch.bfloat16, device=DEV)
    KN.matmul_dgrad(dinp, dout.to(DEV), w.to(DEV))
    ref = torch.empty(M, C)
    R.matmul_dgrad(ref, dout, w)
    close(dinp, ref, 3e-2, 1e-2, "dgrad")


def test_matmul_dgrad_dgelu():
    M, OC, C = 384, 768, 3072
    dout, w, pre = rnd(M, OC), rnd(OC, C, scale=0.05), rnd(M, C)
    dinp = torch.empty(M, C, dtype=torch.bfloat16, device=DEV)
    KN.matmul_dgrad(dinp, dout.to(DEV), w.to(DEV), pre_gelu=pre.to(DEV))
    ref = torch.empty(M, C)
    R.matmul_dgrad(ref, dout, w, pre_gelu=pre)
    close(dinp, ref, 3e-2, 1e-2, "dgrad+dgelu")


@pytest.mark.parametrize("M,OC,C,acc", [(256, 128, 256, False), (4096, 768, 768, True), (2048, 2304, 768, True),
                                          (1000, 264, 136, True), (8192, 256, 512, False),
                                          # two-SM kernel, three K splits, partial tiles in both directions (fold kernel bounds)
                                          (4096, 1600, 1600, True), (2048, 1336, 1544, False)])
def test_matmul_wgrad(M, OC, C, acc):
    dout, inp = rnd(M, OC, scale=0.1), rnd(M, C)
    dw0 = rnd(OC, C)
    dw = dw0.to(DEV).clone()
    KN.matmul_wgrad(dw, dout.to(DEV), inp.to(DEV), accumulate=acc)
    ref = dw0.float().clone()
    R.matmul_wgrad(ref, dout, inp, accumulate=acc)
    close(dw, ref, 5e-2, 1.5e-2, "wgrad")
    # run-twice determinism (split-K folds partials in a fixed order)
    dw2 = dw0.to(DEV).clone()
    KN.matmul_wgrad(dw2, dout.to(DEV), inp.to(DEV), accumulate=acc)
    assert torch.equal(dw, dw2)


def test_bias_grad():
    M, OC = 1000, 776
    dout, db0 = rnd(M, OC), rnd(OC)
    db = db0.to(DEV).clone()
    KN.bias_grad(db, dout.to(DEV), accumulate=True)
    ref = db0.float().clone()
    R.bias_grad(ref, dout, accumulate=True)
    close(db, ref, 5e-2, 1e-2, "bias_grad")


@pytest.mark.parametrize("N,C", [(64, 64), (300, 768), (1031, 768), (128, 1600), (32, 2048 + 512), (257, 4096), (40, 8192)])
def test_layernorm_forward_backward(N, C):
    x, w, b, dy = rnd(N, C), rnd(C) + 1.0, rnd(C), rnd(N, C)
    out = torch.empty(N, C, dtype=torch.bfloat16, device=DEV)
    mean = torch.empty(N, device=DEV)
    rstd = torch.empty(N, device=DEV)
    KN.layernorm_forward(out, mean, rstd, x.to(DEV), w.to(DEV), b.to(DEV))
    ro, rm, rr = torch.empty(N, C), torch.empty(N), torch.empty(N)
    R.layernorm_forward(ro, rm, rr, x, w, b)
    close(out, ro, 2e-2, 1e-2, "ln out")
    close(mean, rm, 1e-4, 1e-4, "ln mean")
    close(rstd, rr, 1e-3, 1e-3, "ln rstd")
    dx0, dw0, db0 = rnd(N, C), rnd(C), rnd(C)
    dx, dw, db = dx0.to(DEV).clone(), dw0.to(DEV).clone(), db0.to(DEV).clone()
    KN.layernorm_backward(dx, dw, db, dy.to(DEV), x.to(DEV), w.to(DEV), mean, rstd, True, True)
    rdx, rdw, rdb = dx0.float().clone(), dw0.float().clone(), db0.float().clone()
    R.layernorm_backward(rdx, rdw, rdb, dy, x, w, rm, rr, True, True)
    close(dx, rdx, 3e-2, 1.5e-2, "ln dx")
    close(dw, rdw, 0.15, 2e-2, "ln dw")
    close(db, rdb, 0.15, 2e-2, "ln db")
    dx2, dw2, db2 = dx0.to(DEV).clone(), dw0.to(DEV).clone(), db0.to(DEV).clone()
    KN.layernorm_backward(dx2, dw2, db2, dy.to(DEV), x.to(DEV), w.to(DEV), mean, rstd, True, True)
    assert torch.equal(dw, dw2) and torch.equal(db, db2) and torch.equal(dx, dx2)
    # fused column sums of the final dinp (the bias gradient of the residual projection), fresh and accumulated
    for acc_col in (False, True):
        dx3, dw3, db3, dc0 = dx0.to(DEV).clone(), dw0.to(DEV).clone(), db0.to(DEV).clone(), rnd(C, seed=21)
        dc = dc0.to(DEV).clone()
        KN.layernorm_backward(dx3, dw3, db3, dy.to(DEV), x.to(DEV), w.to(DEV), mean, rstd, True, True, dcolsum=dc, accumulate_dcol=acc_col)
        assert torch.equal(dx3, dx) and torch.equal(dw3, dw)
        want = dx.float().cpu().sum(0) + (dc0.float() if acc_col else 0.0)
        close(dc, want, 0.2, 2e-2, "ln dcolsum")


def test_fused_residual_forward():
    N, C = 257, 768
    a, b2, w, b = rnd(N, C), rnd(N, C, seed=3), rnd(C) + 1.0, rnd(C)
    res = torch.empty(N, C, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(N, C, dtype=torch.bfloat16, device=DEV)
    mean, rstd = torch.empty(N, device=DEV), torch.empty(N, device=DEV)
    KN.fused_residual_forward(res, out, mean, rstd, a.to(DEV), b2.to(DEV), w.to(DEV), b.to(DEV))
    rres, ro, rm, rr = torch.empty(N, C), torch.empty(N, C), torch.empty(N), torch.empty(N)
    R.fused_residual_forward(rres, ro, rm, rr, a, b2, w, b)
    close(res, rres, 2e-2, 1e-2, "residual")
    close(out, ro, 4e-2, 2e-2, "normed")


def test_encoder_forward_backward():
    B, T, C, V = 4, 64, 768, 1000
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, V, (B, T), generator=g, dtype=torch.int32)
    tok[0, :20] = 5          # heavy collisions
    wte, wpe = rnd(V, C), rnd(T, C)
    out = torch.empty(B, T, C, dtype=torch.bfloat16, device=DEV)
    KN.encoder_forward(out, tok.to(DEV), wte.to(DEV), wpe.to(DEV))
    ro = torch.empty(B, T, C)
    R.encoder_forward(ro, tok, wte, wpe)
    close(out, ro, 2e-2, 1e-2, "encoder fwd")
    dout = rnd(B, T, C)
    dwte0, dwpe0 = rnd(V, C), rnd(T, C)
    dwte, dwpe = dwte0.to(DEV).clone(), dwpe0.to(DEV).clone()
    KN.encoder_backward(dwte, dwpe, dout.to(DEV), tok.to(DEV), True, True, seed=11)
    rwte, rwpe = dwte0.float().clone(), dwpe0.float().clone()
    R.encoder_backward(rwte, rwpe, dout, tok, True, True)
    close(dwte, rwte, 8e-2, 2e-2, "dwte")      # stochastic rounding: one bf16 ulp
    close(dwpe, rwpe, 8e-2, 2e-2, "dwpe")
    dwte2, dwpe2 = dwte0.to(DEV).clone(), dwpe0.to(DEV).clone()
    KN.encoder_backward(dwte2, dwpe2, dout.to(DEV), tok.to(DEV), True, True, seed=11)
    assert torch.equal(dwte, dwte2) and torch.equal(dwpe, dwpe2)


def test_encoder_backward_many_hits():
    """More hits in one 64-id range than the in-kernel list holds: the multi-round path."""
    B, T, C, V = 8, 1024, 64, 200
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, 40, (B, T), generator=g, dtype=torch.int32)
    dout = rnd(B, T, C, scale=0.1)
    dwte = torch.zeros(V, C, dtype=torch.bfloat16, device=DEV)
    dwpe = torch.zeros(T, C, dtype=torch.bfloat16, device=DEV)
    KN.encoder_backward(dwte, dwpe, dout.to(DEV), tok.to(DEV), False, False, seed=3)
    rwte, rwpe = torch.zeros(V, C), torch.zeros(T, C)
    R.encoder_backward(rwte, rwpe, dout, tok, False, False)
    close(dwte, rwte, 0.15, 3e-2, "dwte multi-round")
    close(dwpe, rwpe, 5e-2, 2e-2, "dwpe")


@pytest.mark.parametrize("N,V,Vp", [(64, 1000, 1024), (128, 50257, 50304)])
def test_fused_classifier(N, V, Vp):
    logits = rnd(N, Vp, scale=2.0)
    g = torch.Generator().manual_seed(4)
    tgt = torch.randint(0, V, (N,), generator=g, dtype=torch.int32)
    lg = logits.to(DEV).clone()
    losses = torch.zeros(N, device=DEV)
    KN.fused_classifier(lg, losses, tgt.to(DEV), 1.0 / N, V, True, False)
    rl, rloss = logits.float().clone(), torch.zeros(N)
    R.fused_classifier(rl, rloss, tgt, 1.0 / N, V, True, False)
    close(losses, rloss, 2e-3, 1e-3, "loss")
    close(lg, rl, 1e-4, 2e-2, "dlogits")
    assert (lg[:, V:] == 0).all()


def test_gelu_and_residual():
    n = 8 * 1000
    x, d = rnd(n), rnd(n, seed=5)
    out = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    KN.gelu_forward(out, x.to(DEV))
    ro = torch.empty(n)
    R.gelu_forward(ro, x)
    close(out, ro, 1e-2, 1e-2, "gelu")
    dd = d.to(DEV).clone()
    KN.gelu_backward_inplace(dd, x.to(DEV))
    rd = d.float().clone()
    R.gelu_backward_inplace(rd, x)
    close(dd, rd, 1e-2, 1e-2, "gelu bwd")
    KN.residual_add(out, x.to(DEV), d.to(DEV))
    close(out, x.float() + d.float(), 2e-2, 1e-2, "residual add")


def _views(n, L=1, wd=0.1, seed=123):
    return [dict(p_base=0, p_stride=n // L, o_base=0, o_stride=n // L, n=n // L, L=L, wd=wd, seed=seed)]


def test_global_norm_and_adamw():
    n = 8 * 4096
    p0, g = rnd(n, scale=0.02), rnd(n, scale=0.01, seed=7)
    views = _views(n, L=4)
    out = torch.zeros(1, device=DEV)
    KN.global_norm_sq(out, g.to(DEV), views)
    ref = (g.float() ** 2).sum()
    assert abs(out.item() - ref.item()) <= 1e-4 * ref.item()
    params = p0.to(DEV).clone()
    master = torch.empty(n, device=DEV)
    KN.master_from_params(master, params, views)
    assert torch.equal(master.cpu(), p0.float())
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    nsq = torch.tensor([ref.item()], device=DEV)
    KN.adamw_update(params, master, g.to(DEV), m, v, views, 1e-3, 0.9, 0.95, 1e-8, 1, 1.0, nsq, 0.05)
    rp, rm, rv, rmaster = p0.float().clone(), torch.zeros(n), torch.zeros(n), p0.float().clone()
    R.adamw_update(rp, rmaster, g, rm, rv, views, 1e-3, 0.9, 0.95, 1e-8, 1, 1.0, torch.tensor([ref.item()]), 0.05)
    close(master, rmaster, 1e-6, 1e-5, "master")
    close(m, rm, 1e-7, 1e-5, "m")
    # stochastic rounding: bf16 params within one ulp of the fp32 master and unbiased on average
    diff = params.float().cpu() - master.cpu()
    ulp = master.cpu().abs() * 2.0 ** -7
    assert (diff.abs() <= ulp + 1e-12).all()
    assert abs(diff.mean().item()) < 0.05 * ulp.mean().item()
    # same seeds -> same rounding (resume path)
    p2 = torch.empty_like(params)
    KN.params_from_master(p2, master, views)
    assert torch.equal(p2, params)


@pytest.mark.parametrize("B,T,NH,hs", [(2, 128, 2, 64), (1, 64, 3, 64), (2, 384, 4, 64), (1, 1024, 2, 64), (2, 384, 2, 128), (1, 200, 3, 96),
                                        (2, 256, 2, 80)])
def test_attention_forward(B, T, NH, hs):
    qkv = rnd(B, T, 3 * NH * hs)
    out = torch.full((B, T, NH * hs), float("nan"), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(B, NH, T, device=DEV)
    KN.attention_forward(out, lse, qkv.to(DEV), B, T, NH)
    ro, rl = torch.empty(B, T, NH * hs), torch.empty(B, NH, T)
    R.attention_forward(ro, rl, qkv, B, T, NH)
    close(lse, rl, 2e-2, 1e-3, "lse")
    close(out, ro, 2e-2, 2e-2, "attention out")


@pytest.mark.parametrize("B,T,NH,hs", [(1, 128, 1, 64), (2, 64, 2, 64), (2, 384, 3, 64), (1, 1024, 2, 64), (2, 384, 2, 128), (1, 200, 3, 96),
                                        (2, 256, 2, 80)])
def test_attention_backward(B, T, NH, hs):
    qkv = rnd(B, T, 3 * NH * hs)
    dout = rnd(B, T, NH * hs, scale=0.5, seed=9)
    dev_qkv = qkv.to(DEV)
    out = torch.empty(B, T, NH * hs, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(B, NH, T, device=DEV)
    KN.attention_forward(out, lse, dev_qkv, B, T, NH)
    dqkv = torch.full((B, T, 3 * NH * hs), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.attention_backward(dqkv, dout.to(DEV), dev_qkv, out, lse, B, T, NH)
    ro, rl = torch.empty(B, T, NH * hs), torch.empty(B, NH, T)
    R.attention_forward(ro, rl, qkv, B, T, NH)
    rd = torch.empty(B, T, 3 * NH * hs)
    R.attention_backward(rd, dout, qkv, ro, rl, B, T, NH)
    close(dqkv, rd, 4e-2, 3e-2, "dqkv")
    dqkv2 = torch.empty_like(dqkv)
    KN.attention_backward(dqkv2, dout.to(DEV), dev_qkv, out, lse, B, T, NH)
    assert torch.equal(dqkv, dqkv2)


@pytest.mark.parametrize("M,N,K", [(512, 512, 128), (1024, 2304, 768), (300, 520, 320), (2048, 768, 3072)])
def test_two_sm_gemm_forward_and_dgrad(M, N, K, monkeypatch):
    """The cta_group::2 kernel (256 x 256 tiles on CTA pairs) against the fp32 reference, all of its epilogues."""
    monkeypatch.setattr(KN, "TWO_SM_MIN_TILES", 1)
    inp, w, b = rnd(M, K), rnd(N, K, scale=0.05), rnd(N)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.matmul_forward(out, inp.to(DEV), w.to(DEV), b.to(DEV))
    ref = torch.empty(M, N)
    R.matmul_forward(ref, inp, w, b)
    close(out, ref, 2e-2, 1e-2, "2sm forward")
    pre = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    KN.matmul_forward(out, inp.to(DEV), w.to(DEV), b.to(DEV), pre_gelu=pre)
    refpre = torch.empty(M, N)
    R.matmul_forward(ref, inp, w, b, pre_gelu=refpre)
    close(pre, refpre, 2e-2, 1e-2, "2sm pre-gelu")
    close(out, ref, 2e-2, 1e-2, "2sm gelu")
    # dgrad: dinp[M,K] = dout[M,N] @ w[N,K] (B operand MN-major), with and without dGELU
    dout = rnd(M, N, seed=3)
    dinp = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    KN.matmul_dgrad(dinp, dout.to(DEV), w.to(DEV))
    rd = torch.empty(M, K)
    R.matmul_dgrad(rd, dout, w)
    close(dinp, rd, 3e-2, 1e-2, "2sm dgrad")
    pg = rnd(M, K, seed=5)
    KN.matmul_dgrad(dinp, dout.to(DEV), w.to(DEV), pre_gelu=pg.to(DEV))
    R.matmul_dgrad(rd, dout, w, pre_gelu=pg)
    close(dinp, rd, 3e-2, 1e-2, "2sm dgrad+dgelu")


@pytest.mark.parametrize("M,N,K,acc,use_bias", [(128, 128, 32, False, False), (256, 384, 768, False, True), (200, 132, 100, True, False),
                                                (1024, 768, 3072, True, True), (64, 50304 // 8, 768, False, False)])
def test_gemm_tf32(M, N, K, acc, use_bias):
    """The full-precision mode's matmul: fp32 in memory, TF32 products (10-bit mantissa inputs), fp32 accumulation."""
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(N, K, generator=g) * 0.05
    bias = torch.randn(N, generator=g) if use_bias else None
    d0 = torch.randn(M, N, generator=g)
    buf = torch.full((M + 4, N), 7.0, device=DEV)
    buf[:M].copy_(d0)
    KN.gemm_tf32(buf[:M], a.to(DEV), b.to(DEV), None if bias is None else bias.to(DEV), accumulate=acc)
    ref = a.double() @ b.double().t()
    if bias is not None:
        ref = ref + bias.double()
    if acc:
        ref = ref + d0.double()
    # TF32 keeps 10 mantissa bits of each input (truncated, not rounded): per-product relative error up to 2^-9, summed over K
    # terms of magnitude ~ |a| |b| = 0.05; the factor covers the tail of the maximum over all outputs
    tol = 2.0 ** -9 * math.sqrt(K) * 0.05 * 4.0 + 1e-5
    err = (buf[:M].double().cpu() - ref).abs().max().item()
    assert err < tol, "max err %g (tolerance %g)" % (err, tol)
    assert (buf[M:] == 7.0).all()
