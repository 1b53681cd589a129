"""End-to-end numerics of the hand-written forward/backward against an autograd oracle (the scheme of the
reference's test_gpt2.c: logits, loss, all 16 gradient tensors, then a few optimizer steps)."""
import math

import pytest
import torch

from llmc_b200.models import gpt2
from llmc_b200.parallel.dist import DistConfig
from llmc_b200.parallel.zero import ShardedAdamW
from oracle import oracle_loss_and_grads


def small_model(recompute=0, dtype=torch.float32, L=2):
    cfg = gpt2.GPTConfig(max_seq_len=32, vocab_size=97, padded_vocab_size=104, num_layers=L, num_heads=2, channels=32)
    m = gpt2.GPT(cfg, "cpu", dtype, recompute=recompute)
    m.init_random(42)
    # give biases and LayerNorm parameters non-trivial values so their gradients are exercised
    g = torch.Generator().manual_seed(1)
    for n in ("ln1b", "qkvb", "attprojb", "ln2b", "fcb", "fcprojb", "lnfb"):
        m.params[n].copy_(torch.randn(m.params[n].shape, generator=g) * 0.1)
    for n in ("ln1w", "ln2w", "lnfw"):
        m.params[n].add_(torch.randn(m.params[n].shape, generator=g) * 0.1)
    return m


def batch(cfg, B=3, T=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


@pytest.mark.parametrize("recompute", [0, 1, 2])
def test_forward_backward_matches_autograd(recompute):
    m = small_model(recompute)
    x, y = batch(m.cfg)
    ref_logits, ref_loss, ref_grads = oracle_loss_and_grads(m, x, y)
    m.forward(x, y, write_dlogits=False)
    B, T = x.shape
    logits = m.logits()[..., :m.cfg.vocab_size]
    assert torch.allclose(logits, ref_logits[..., :m.cfg.vocab_size], atol=1e-4, rtol=1e-4)
    m.forward(x, y)
    m.backward()
    assert abs(float(m.loss()) - ref_loss) < 1e-4
    for name in gpt2.PARAM_NAMES:
        got, want = m.grads[name], ref_grads[name]
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), "gradient of %s: max err %g" % (name, (got - want).abs().max())


def test_gradient_accumulation_equals_big_batch():
    m = small_model()
    x, y = batch(m.cfg, B=4)
    m.forward(x, y)
    m.backward()
    full = m.grads_flat.clone()
    for micro in range(2):
        m.forward(x[2 * micro:2 * micro + 2], y[2 * micro:2 * micro + 2], grad_accum_steps=2, micro_step=micro)
        m.backward(micro, last_micro_step=(micro == 1))
    assert torch.allclose(m.grads_flat, full, atol=1e-5, rtol=1e-4)
    assert abs(float(m.loss(2)) - float(torch.nn.functional.cross_entropy(
        oracle_loss_and_grads(m, x, y)[0][..., :m.cfg.vocab_size].reshape(-1, m.cfg.vocab_size), y.reshape(-1).long()))) < 1e-4


def test_overfit_single_batch_loss_decreases():
    """The correctness anchor of the reference (test_gpt2.c:89-100): ten AdamW steps on one batch."""
    m = small_model(L=2)
    opt = ShardedAdamW(m, DistConfig(), 0, False, beta2=0.999, grad_clip=1e9)
    x, y = batch(m.cfg, B=4, T=16)
    losses = []
    for step in range(10):
        m.forward(x, y)
        m.backward()
        losses.append(float(m.loss()))
        opt.grad_norm_sq()
        opt.step(3e-3, 0.0, step + 1)
    assert losses[0] > math.log(m.cfg.vocab_size) - 0.5
    assert all(b < a for a, b in zip(losses, losses[1:])), losses
    assert losses[-1] < losses[0] - 0.5, losses


def test_descriptors_and_parameter_count():
    cfg = gpt2.config_from_descriptor("d12")
    assert (cfg.num_layers, cfg.num_heads, cfg.channels, cfg.max_seq_len) == (12, 12, 768, 1024)
    assert gpt2.num_parameters(cfg) == 124475904          # padded vocabulary (50304 rows)
    assert gpt2.config_from_descriptor("gpt2:d48").channels == 1600
    g3 = gpt2.config_from_descriptor("gpt3:c768")
    assert (g3.max_seq_len, g3.num_layers) == (2048, 12)
    with pytest.raises(ValueError):
        gpt2.config_from_descriptor("x9")


def test_init_matches_torch_module_init_order():
    """One mt19937 normal stream, consumed in module order: wte, wpe, then per layer qkvw, attprojw, fcw, fcprojw."""
    cfg = gpt2.GPTConfig(max_seq_len=8, vocab_size=20, padded_vocab_size=24, num_layers=2, num_heads=2, channels=16)
    m = gpt2.GPT(cfg, "cpu", torch.float32)
    m.init_random(42)
    g = torch.Generator().manual_seed(42)
    wte = torch.empty(20, 16).normal_(0, 0.02, generator=g)
    wpe = torch.empty(8, 16).normal_(0, 0.02, generator=g)
    qkv0 = torch.empty(48, 16).normal_(0, 0.02, generator=g)
    proj0 = torch.empty(16, 16).normal_(0, 0.02 / math.sqrt(4), generator=g)
    assert torch.allclose(m.params["wte"][:20], wte, atol=1e-7)
    assert (m.params["wte"][20:] == 0).all()
    assert torch.allclose(m.params["wpe"], wpe, atol=1e-7)
    assert torch.allclose(m.params["qkvw"][0], qkv0, atol=1e-7)
    assert torch.allclose(m.params["attprojw"][0], proj0, atol=1e-7)
    assert (m.params["ln1w"] == 1).all() and (m.params["qkvb"] == 0).all()
