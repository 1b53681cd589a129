"""The bf16 sm_100a path against the fp32 CPU path of the same model code (the scheme of the reference's test_gpt2.cu:
logits, loss, per-tensor gradients with bf16 tolerances, a few optimizer steps, and bit-exact determinism)."""
import math

import pytest
import torch

from llmc_b200.models import gpt2
from llmc_b200.parallel.dist import DistConfig
from llmc_b200.parallel.zero import ShardedAdamW

pytestmark = pytest.mark.gpu


def make(device, dtype, recompute=0, L=2, C=128, NH=2, T=128, V=1000, Vp=1024):
    cfg = gpt2.GPTConfig(max_seq_len=T, vocab_size=V, padded_vocab_size=Vp, num_layers=L, num_heads=NH, channels=C)
    m = gpt2.GPT(cfg, device, dtype, recompute=recompute)
    m.init_random(42)
    return m


def batch(cfg, B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


@pytest.mark.parametrize("recompute,T", [(0, 128), (1, 64), (2, 128)])
def test_gpu_matches_cpu_reference(recompute, T):
    gm = make("cuda", torch.bfloat16, recompute)
    cm = make("cpu", torch.float32, recompute)
    cm.params_flat.copy_(gm.params_flat.float().cpu())          # identical (bf16-representable) parameters
    x, y = batch(gm.cfg, 4, T)
    cm.forward(x, y, write_dlogits=False)
    gm.forward(x.cuda(), y.cuda(), write_dlogits=False)
    V = gm.cfg.vocab_size
    lg, lc = gm.logits()[..., :V].float().cpu(), cm.logits()[..., :V]
    assert (lg - lc).abs().max() < 0.05 + 0.02 * lc.abs().max(), (lg - lc).abs().max()
    cm.forward(x, y)
    cm.backward()
    gm.forward(x.cuda(), y.cuda())
    gm.backward()
    assert abs(float(gm.loss()) - float(cm.loss())) < 2e-2
    for name in gpt2.PARAM_NAMES:
        got, want = gm.grads[name].float().cpu(), cm.grads[name]
        scale = want.abs().max().item() + 1e-6
        err = (got - want).abs().max().item()
        assert err < 0.06 * scale + 1e-4, "gradient of %s: max err %g vs max %g" % (name, err, scale)


def test_gpu_training_reduces_loss_and_is_deterministic():
    runs = []
    for _ in range(2):
        m = make("cuda", torch.bfloat16, 0)
        opt = ShardedAdamW(m, DistConfig(0, 1, 0, torch.device("cuda", 0)), 0, True)
        x, y = batch(m.cfg, 4, 128)
        x, y = x.cuda(), y.cuda()
        losses = []
        for step in range(8):
            for micro in range(2):
                m.forward(x[2 * micro:2 * micro + 2].contiguous(), y[2 * micro:2 * micro + 2].contiguous(), 2, micro)
                m.backward(micro, micro == 1)
            losses.append(float(m.loss(2)))
            opt.grad_norm_sq()
            opt.step(3e-3, 0.1, step + 1)
        runs.append((losses, m.params_flat.clone()))
    l0, p0 = runs[0]
    l1, p1 = runs[1]
    assert l0[0] > math.log(1000) - 0.5 and l0[-1] < l0[0] - 0.5, l0
    assert l0 == l1 and torch.equal(p0, p1), "two identical runs must agree bit for bit"


@pytest.mark.parametrize("C,NH", [(256, 2), (192, 2), (160, 2)])
def test_gpu_matches_cpu_reference_wide_heads(C, NH):
    """Head sizes 128, 96 and 80 (the GPT-3 family) run on the 128-wide attention kernels."""
    gm = make("cuda", torch.bfloat16, 0, L=2, C=C, NH=NH, T=256)
    cm = make("cpu", torch.float32, 0, L=2, C=C, NH=NH, T=256)
    cm.params_flat.copy_(gm.params_flat.float().cpu())
    x, y = batch(gm.cfg, 2, 200)
    cm.forward(x, y)
    cm.backward()
    gm.forward(x.cuda(), y.cuda())
    gm.backward()
    assert abs(float(gm.loss()) - float(cm.loss())) < 2e-2
    for name in gpt2.PARAM_NAMES:
        got, want = gm.grads[name].float().cpu(), cm.grads[name]
        scale = want.abs().max().item() + 1e-6
        assert (got - want).abs().max().item() < 0.06 * scale + 1e-4, name


def test_fp32_mode_on_the_gpu_matches_the_cpu_path():
    """The legacy full-precision mode (all tensors fp32 on the device) follows the CPU path to fp32 round-off."""
    torch.backends.cuda.matmul.allow_tf32 = False
    gm = make("cuda", torch.float32, 1)
    cm = make("cpu", torch.float32, 1)
    assert torch.equal(gm.params_flat.cpu(), cm.params_flat)
    x, y = batch(gm.cfg, 2, 64)
    for m, dev in ((gm, "cuda"), (cm, "cpu")):
        m.forward(x.to(dev), y.to(dev))
        m.backward()
    assert abs(float(gm.loss()) - float(cm.loss())) < 1e-4
    assert torch.allclose(gm.grads_flat.cpu(), cm.grads_flat, atol=1e-4, rtol=1e-3)
    opt = ShardedAdamW(gm, DistConfig(0, 1, 0, torch.device("cuda", 0)), 0, True)
    assert opt.master is None
    before = gm.params_flat.clone()
    opt.grad_norm_sq()
    opt.step(1e-3, 0.1, 1)
    assert not torch.equal(before, gm.params_flat) and torch.isfinite(gm.params_flat).all()


def test_fp32_mode_with_tf32_kernel_tracks_the_cpu_path():
    """With TF32 allowed the matmuls of the full-precision mode run on this library's kind::tf32 kernel."""
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        gm = make("cuda", torch.float32, 0)
        cm = make("cpu", torch.float32, 0)
        x, y = batch(gm.cfg, 2, 64)
        from llmc_b200.ops import kernels as KN
        before = KN.launch_count()
        for m, dev in ((gm, "cuda"), (cm, "cpu")):
            m.forward(x.to(dev), y.to(dev))
            m.backward()
        assert KN.launch_count() - before >= 3 * (4 * gm.cfg.num_layers + 1)      # every matmul went through llmc_gemm_tf32
        assert abs(float(gm.loss()) - float(cm.loss())) < 5e-3
        for name in gpt2.PARAM_NAMES:
            got, want = gm.grads[name].cpu(), cm.grads[name]
            scale = want.abs().max().item() + 1e-6
            assert (got - want).abs().max().item() < 0.02 * scale + 1e-5, name
    finally:
        torch.backends.cuda.matmul.allow_tf32 = False


def test_optimizer_state_in_managed_memory_trains_identically(monkeypatch):
    """The fallback placement of the AdamW moments and master weights (managed memory that prefers the host) changes where the
    state lives, not what the update computes."""
    runs = []
    for force in ("0", "1"):
        monkeypatch.setenv("LLMC_FORCE_MANAGED", force)
        m = make("cuda", torch.bfloat16, 0)
        opt = ShardedAdamW(m, DistConfig(0, 1, 0, torch.device("cuda", 0)), 0, True)
        assert opt.state_in_managed_memory == (force == "1")
        x, y = batch(m.cfg, 2, 128)
        x, y = x.cuda(), y.cuda()
        for step in range(3):
            m.forward(x, y)
            m.backward()
            opt.grad_norm_sq()
            opt.step(3e-3, 0.1, step + 1)
        torch.cuda.synchronize()
        runs.append((m.params_flat.clone(), opt.m.clone(), opt.master.clone()))
        del opt, m
    for a, b in zip(runs[0], runs[1]):
        assert torch.equal(a, b)
