"""Every full-precision kernel (csrc/fp32_ops.cu through ops/kernels_fp32.py) against the plain PyTorch restatement of the same
operator on the same device tensors (the scheme of the reference's dev/cuda/*.cu mains: CPU / library result vs kernel)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a GPU", allow_module_level=True)

from llmc_b200 import _lib
from llmc_b200.ops import kernels_fp32 as K
from llmc_b200.ops import reference as R

DEV = "cuda"


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(DEV)


def close(a, b, tol=1e-5):
    scale = max(float(b.abs().max()), 1e-6)
    err = float((a - b).abs().max()) / scale
    assert err < tol, "relative error %.3g" % err


@pytest.fixture(autouse=True)
def _ieee_fp32():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old
    assert _lib.read_status() == 0


def test_elementwise():
    x, d = rnd(1000, 768, scale=2.0), rnd(1000, 768, seed=1)
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    K.gelu_forward(o1, x); R.gelu_forward(o2, x); close(o1, o2)
    d1, d2 = d.clone(), d.clone()
    K.gelu_backward_inplace(d1, x); R.gelu_backward_inplace(d2, x); close(d1, d2)
    K.residual_add(o1, x, d); close(o1, x + d)


@pytest.mark.parametrize("C", [768, 1600])
def test_encoder(C):
    B, T, V = 4, 64, 1000
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, V, (B, T), generator=g, dtype=torch.int32).to(DEV)
    tokens[0, :8] = 5                                     # collisions on one id
    wte, wpe = rnd(V, C), rnd(T, C, seed=1)
    o1, o2 = torch.empty(B, T, C, device=DEV), torch.empty(B, T, C, device=DEV)
    K.encoder_forward(o1, tokens, wte, wpe); R.encoder_forward(o2, tokens, wte, wpe); close(o1, o2, 1e-7)
    dout = rnd(B, T, C, seed=2)
    for acc in (False, True):
        a1, a2 = rnd(V, C, seed=4), rnd(T, C, seed=5)
        b1, b2 = a1.clone(), a2.clone()
        K.encoder_backward(a1, a2, dout, tokens, acc, acc); R.encoder_backward(b1, b2, dout, tokens, acc, acc)
        close(a1, b1); close(a2, b2)
    a1, b1 = rnd(V, C, seed=4), None
    b1 = a1.clone()
    K.encoder_backward(a1, None, dout, tokens, True, True); R.encoder_backward(b1, None, dout, tokens, True, True); close(a1, b1)


@pytest.mark.parametrize("rows,C", [(515, 768), (130, 1600), (64, 2880)])
def test_layernorm(rows, C):
    x, x2, w, b = rnd(rows, C, scale=2.0), rnd(rows, C, seed=1), rnd(C, seed=2), rnd(C, seed=3)
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    m1, r1, m2, r2 = (torch.empty(rows, device=DEV) for _ in range(4))
    K.layernorm_forward(o1, m1, r1, x, w, b); R.layernorm_forward(o2, m2, r2, x, w, b)
    close(o1, o2); close(m1, m2); close(r1, r2)
    K.layernorm_forward(o1, None, None, x, w, b); close(o1, o2)
    res1, res2 = torch.empty_like(x), torch.empty_like(x)
    K.fused_residual_forward(res1, o1, m1, r1, x, x2, w, b); R.fused_residual_forward(res2, o2, m2, r2, x, x2, w, b)
    close(res1, res2, 1e-7); close(o1, o2); close(r1, r2)
    dy = rnd(rows, C, seed=4)
    for acc_i, acc_w, col, acc_c in [(False, False, False, False), (True, True, True, True), (True, False, True, False)]:
        di1, dw1, db1, dc1 = rnd(rows, C, seed=5), rnd(C, seed=6), rnd(C, seed=7), rnd(C, seed=8)
        di2, dw2, db2, dc2 = di1.clone(), dw1.clone(), db1.clone(), dc1.clone()
        K.layernorm_backward(di1, dw1, db1, dy, res1, w, m1, r1, acc_i, acc_w, dc1 if col else None, acc_c)
        R.layernorm_backward(di2, dw2, db2, dy, res2, w, m2, r2, acc_i, acc_w, dc2 if col else None, acc_c)
        close(di1, di2, 2e-5); close(dw1, dw2, 2e-5); close(db1, db2, 2e-5); close(dc1, dc2, 2e-5)


@pytest.mark.parametrize("rows,OC", [(1000, 768), (77, 2304)])
def test_bias_grad(rows, OC):
    d = rnd(rows, OC)
    for acc in (False, True):
        a = rnd(OC, seed=1)
        b = a.clone()
        K.bias_grad(a, d, acc); R.bias_grad(b, d, acc); close(a, b)


def test_classifier():
    N, V, Vp = 96, 1000, 1024
    logits = rnd(N, Vp, scale=3.0)
    g = torch.Generator().manual_seed(1)
    targets = torch.randint(0, V, (N,), generator=g, dtype=torch.int32).to(DEV)
    for write, acc in [(True, False), (False, True)]:
        l1, l2 = logits.clone(), logits.clone()
        s1 = rnd(N, seed=2)
        s2 = s1.clone()
        K.fused_classifier(l1, s1, targets, 0.25, V, write, acc); R.fused_classifier(l2, s2, targets, 0.25, V, write, acc)
        close(s1, s2); close(l1, l2)


@pytest.mark.parametrize("B,T,NH,hs", [(2, 128, 3, 64), (1, 200, 2, 32)])
def test_attention(B, T, NH, hs):
    qkv = rnd(B, T, 3 * NH * hs)
    o1, o2 = torch.empty(B, T, NH * hs, device=DEV), torch.empty(B, T, NH * hs, device=DEV)
    l1, l2 = torch.empty(B, NH, T, device=DEV), torch.empty(B, NH, T, device=DEV)
    K.attention_forward(o1, l1, qkv, B, T, NH); R.attention_forward(o2, l2, qkv, B, T, NH)
    close(o1, o2); close(l1, l2)
    dout = rnd(B, T, NH * hs, seed=1)
    d1, d2 = torch.empty_like(qkv), torch.empty_like(qkv)
    K.attention_backward(d1, dout, qkv, o1, l1, B, T, NH); R.attention_backward(d2, dout, qkv, o2, l2, B, T, NH)
    close(d1, d2, 2e-5)


def test_optimizer_and_norm():
    n, L = 1000, 3
    views = [dict(name="a", p_base=0, p_stride=n, o_base=0, o_stride=n, n=n, L=L, wd=0.1, seed=0),
             dict(name="b", p_base=L * n, p_stride=0, o_base=L * n, o_stride=0, n=520, L=1, wd=0.0, seed=0)]
    total = L * n + 520
    for use_master in (False, True):
        p1, g, m1, v1 = rnd(total), rnd(total, seed=1, scale=0.1), rnd(total, seed=2, scale=0.01), rnd(total, seed=3, scale=0.01).abs()
        p2, m2, v2 = p1.clone(), m1.clone(), v1.clone()
        ma1 = p1.clone() if use_master else None
        ma2 = p2.clone() if use_master else None
        ns1, ns2 = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
        K.global_norm_sq(ns1, g, views); R.global_norm_sq(ns2, g, views); close(ns1, ns2)
        K.adamw_update(p1, ma1, g, m1, v1, views, 1e-3, 0.9, 0.95, 1e-8, 3, 1.0, ns1, 1.0)
        R.adamw_update(p2, ma2, g, m2, v2, views, 1e-3, 0.9, 0.95, 1e-8, 3, 1.0, ns2, 1.0)
        close(p1, p2); close(m1, m2); close(v1, v2)
        if use_master:
            close(ma1, ma2)
            q1, q2 = torch.zeros_like(p1), torch.zeros_like(p1)
            K.params_from_master(q1, ma1, views); R.params_from_master(q2, ma2, views); close(q1, q2, 1e-7)
            K.master_from_params(ma1, p2 * 2, views); R.master_from_params(ma2, p2 * 2, views); close(ma1, ma2, 1e-7)
    # a non-finite norm skips the update
    p1 = rnd(total)
    before = p1.clone()
    K.adamw_update(p1, None, rnd(total, seed=1), torch.zeros(total, device=DEV), torch.zeros(total, device=DEV), views, 1e-3, 0.9, 0.95, 1e-8, 1,
                   1.0, torch.full((1,), float("inf"), device=DEV), 1.0)
    assert torch.equal(p1, before)
