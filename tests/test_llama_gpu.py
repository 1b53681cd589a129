"""LLaMA-3 family on a B200: each new kernel against the PyTorch fp32 restatement of the same operator, then the whole
bf16 model against the fp32 CPU path of the same model code (logits, loss, every gradient tensor), training and
bit-exact determinism."""
import math

import pytest
import torch

from llmc_b200.models import llama3
from llmc_b200.ops import kernels as KN
from llmc_b200.ops import reference as R
from llmc_b200.parallel.dist import DistConfig
from llmc_b200.parallel.zero import ShardedAdamW

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, scale=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, atol, rtol, what):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    bad = (err > atol + rtol * want.abs()).sum().item()
    assert bad == 0, "%s: %d/%d elements off, max err %.4g (max ref %.4g)" % (what, bad, err.numel(), err.max().item(), want.abs().max().item())


@pytest.mark.parametrize("N,C", [(64, 64), (300, 768), (257, 2048), (130, 4096), (40, 8192), (24, 16384)])
def test_rmsnorm_forward_backward(N, C):
    x, x2, w, dy = rnd(N, C), rnd(N, C, seed=1), (1.0 + 0.2 * rnd(C, seed=2).float()).to(torch.bfloat16), rnd(N, C, seed=3)
    out = torch.empty(N, C, dtype=torch.bfloat16, device=DEV)
    rstd = torch.empty(N, dtype=torch.float32, device=DEV)
    KN.rmsnorm_forward(out, rstd, x.to(DEV), w.to(DEV), 1e-5)
    ro, rr = torch.empty(N, C, dtype=torch.bfloat16), torch.empty(N)
    R.rmsnorm_forward(ro, rr, x, w, 1e-5)
    close(out, ro, 2e-2, 1e-2, "rmsnorm fwd")
    close(rstd, rr, 1e-5, 1e-4, "rmsnorm rstd")
    # fused residual
    res = torch.empty(N, C, dtype=torch.bfloat16, device=DEV)
    KN.rmsnorm_fused_residual_forward(res, out, rstd, x.to(DEV), x2.to(DEV), w.to(DEV), 1e-5)
    rres = torch.empty(N, C, dtype=torch.bfloat16)
    R.rmsnorm_fused_residual_forward(rres, ro, rr, x, x2, w, 1e-5)
    assert torch.equal(res.cpu(), rres)
    close(out, ro, 3e-2, 1e-2, "fused rmsnorm fwd")
    close(rstd, rr, 1e-5, 1e-4, "fused rmsnorm rstd")
    # backward, both accumulate settings
    for acc in (False, True):
        dx0, dw0 = rnd(N, C, seed=5), rnd(C, seed=6)
        dx, dw = dx0.to(DEV).clone(), dw0.to(DEV).clone()
        KN.rmsnorm_backward(dx, dw, dy.to(DEV), rres.to(DEV), w.to(DEV), rstd, accumulate_dinp=acc, accumulate_dw=acc)
        rdx, rdw = dx0.float().clone(), dw0.float().clone()
        R.rmsnorm_backward(rdx, rdw, dy, rres, w, rr, accumulate_dinp=acc, accumulate_dw=acc)
        close(dx, rdx, 3e-2, 2e-2, "rmsnorm dinp acc=%s" % acc)
        close(dw, rdw, 0.02 * math.sqrt(N) + 0.05, 2e-2, "rmsnorm dweight acc=%s" % acc)
        dx2, dw2 = dx0.to(DEV).clone(), dw0.to(DEV).clone()
        KN.rmsnorm_backward(dx2, dw2, dy.to(DEV), rres.to(DEV), w.to(DEV), rstd, accumulate_dinp=acc, accumulate_dw=acc)
        assert torch.equal(dx, dx2) and torch.equal(dw, dw2)


@pytest.mark.parametrize("B,T,NH,NKV,HS", [(2, 64, 4, 2, 64), (1, 128, 8, 8, 64), (3, 32, 8, 2, 128), (2, 16, 6, 1, 96)])
def test_rope_forward_backward(B, T, NH, NKV, HS):
    cfg = llama3.LlamaConfig(max_seq_len=2 * T, num_heads=NH, num_kv_heads=NKV, channels=NH * HS)
    freqs = llama3.rope_table(cfg)
    N, QR = B * T, (NH + 2 * NKV) * HS
    raw = rnd(N, QR)
    packed = torch.full((N, 3 * NH * HS), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.rope_forward(packed, raw.to(DEV), freqs.to(DEV), T, NH, NKV)
    ref = torch.empty(N, 3 * NH * HS, dtype=torch.bfloat16)
    R.rope_forward(ref, raw, freqs, T, NH, NKV)
    close(packed, ref, 1e-2, 1e-2, "rope fwd")
    dpacked = rnd(N, 3 * NH * HS, seed=4)
    draw = torch.full((N, QR), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.rope_backward(draw, dpacked.to(DEV), freqs.to(DEV), T, NH, NKV)
    rdraw = torch.empty(N, QR)
    R.rope_backward(rdraw, dpacked, freqs, T, NH, NKV)
    close(draw, rdraw, 2e-2, 1e-2, "rope bwd")


@pytest.mark.parametrize("N,H", [(64, 64), (300, 1032), (129, 14336)])
def test_swiglu_forward_backward(N, H):
    x12, dh = rnd(N, 2 * H, scale=2.0), rnd(N, H, seed=3)
    h = torch.empty(N, H, dtype=torch.bfloat16, device=DEV)
    KN.swiglu_forward(h, x12.to(DEV))
    rh = torch.empty(N, H)
    R.swiglu_forward(rh, x12)
    close(h, rh, 2e-2, 1e-2, "swiglu fwd")
    dx = torch.full((N, 2 * H), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.swiglu_backward(dx, dh.to(DEV), x12.to(DEV))
    rdx = torch.empty(N, 2 * H)
    R.swiglu_backward(rdx, dh, x12)
    close(dx, rdx, 3e-2, 1e-2, "swiglu bwd")


def test_encoder_without_position_table():
    B, T, C, V = 2, 64, 128, 300
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, V, (B, T), generator=g, dtype=torch.int32)
    wte, dout = rnd(V, C), rnd(B, T, C, seed=2)
    out = torch.empty(B, T, C, dtype=torch.bfloat16, device=DEV)
    KN.encoder_forward(out, tok.to(DEV), wte.to(DEV), None)
    assert torch.equal(out.cpu(), wte[tok.long()])
    dwte = torch.full((V, C), 3.0, dtype=torch.bfloat16, device=DEV)
    KN.encoder_backward(dwte, None, dout.to(DEV), tok.to(DEV), accumulate_wte=False, accumulate_wpe=False, seed=1)
    ref = torch.zeros(V, C)
    R.encoder_backward(ref, None, dout, tok, accumulate_wte=False, accumulate_wpe=False)
    close(dwte, ref, 5e-2, 2e-2, "encoder bwd without wpe")


def make(device, dtype, recompute=0, desc="llama3:l=2,c=256,h=4,kv=2,t=128,v=1000,m=128,f=1.0"):
    m = llama3.Llama(llama3.config_from_descriptor(desc), device, dtype, recompute=recompute)
    m.init_random(42)
    return m


def batch(cfg, B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


@pytest.mark.parametrize("recompute,desc", [(0, "llama3:l=2,c=256,h=4,kv=2,t=128,v=1000,m=128,f=1.0"),
                                            (1, "llama3:l=2,c=256,h=2,kv=1,t=128,v=1000,m=64,f=1.3"),
                                            (2, "llama3:l=2,c=192,h=2,kv=2,t=128,v=1000,m=128,f=1.0")])
def test_gpu_matches_cpu_reference(recompute, desc):
    gm = make("cuda", torch.bfloat16, recompute, desc)
    cm = make("cpu", torch.float32, recompute, desc)
    cm.params_flat.copy_(gm.params_flat.float().cpu())
    x, y = batch(gm.cfg, 4, 128)
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
    for name in llama3.PARAM_NAMES:
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


@pytest.mark.parametrize("B,Tq,start,Tmax,NH,NKV,HS", [(2, 5, 0, 16, 4, 2, 64), (3, 1, 700, 1024, 8, 2, 128), (1, 9, 40, 64, 6, 3, 96),
                                                       (2, 3, 5, 16, 4, 4, 64), (1, 2, 1100, 1200, 2, 1, 64),
                                                       # the split-key decoding kernel: 8, 1 and 2 query rows per cached head, many slices
                                                       (2, 2, 300, 1024, 8, 2, 128), (2, 1, 50, 512, 4, 4, 64), (1, 1, 1900, 2048, 4, 2, 64)])
def test_decoding_kernels(B, Tq, start, Tmax, NH, NKV, HS):
    """Rotary embedding into the cache and attention over the cache against the fp32 restatement (also beyond one 512-key
    chunk of the running softmax)."""
    cfg = llama3.LlamaConfig(max_seq_len=Tmax, num_heads=NH, num_kv_heads=NKV, channels=NH * HS)
    freqs = llama3.rope_table(cfg)
    N, QR = B * Tq, (NH + 2 * NKV) * HS
    raw = rnd(N, QR)
    kc, vc = rnd(B, Tmax, NKV, HS, seed=1), rnd(B, Tmax, NKV, HS, seed=2)
    rq, rk, rv = torch.zeros(N, NH * HS), kc.float().clone(), vc.float().clone()
    R.rope_cache(rq, rk, rv, raw, freqs, Tq, start, NH, NKV)
    q = torch.zeros(N, NH * HS, dtype=torch.bfloat16, device=DEV)
    dk, dv = kc.to(DEV), vc.to(DEV)
    KN.rope_cache(q, dk, dv, raw.to(DEV), freqs.to(DEV), Tq, start, NH, NKV)
    close(q, rq, 2e-2, 1e-2, "rope_cache q")
    close(dk, rk, 2e-2, 1e-2, "rope_cache k")
    assert torch.equal(dv.cpu()[:, start:start + Tq], raw.view(B, Tq, NH + 2 * NKV, HS)[:, :, NH + NKV:])
    assert torch.equal(dv.cpu()[:, :start], vc[:, :start])                 # nothing else is touched
    ro = torch.zeros(N, NH * HS)
    R.cached_attention(ro, q.cpu(), dk.cpu(), dv.cpu(), Tq, start, NH, NKV)
    out = torch.full((N, NH * HS), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.cached_attention(out, q, dk, dv, Tq, start, NH, NKV)
    close(out, ro, 2e-2, 2e-2, "cached_attention")


def test_cached_decoder_and_generate():
    """The bf16 decoder on the GPU against the fp32 CPU decoder over the same (bf16-rounded) weights, and generation with the
    cache against generation that recomputes the prefix."""
    from llmc_b200.models import generate as G
    cfg = llama3.config_from_descriptor("llama3:l=2,c=256,h=4,kv=2,t=128,v=500,m=64,f=1.0")
    m = llama3.Llama(cfg, DEV, torch.bfloat16, recompute=1)
    m.init_random(3)
    for n in ("qkvw", "attprojw", "fc12w", "fcprojw"):
        m.params[n].mul_(3.0)
    c = llama3.Llama(cfg, "cpu", torch.float32, recompute=0)
    c.params_flat.copy_(m.params_flat.float().cpu())
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (3, 40), generator=g, dtype=torch.int32)
    dm, dc = G.CachedDecoder(m, 3, 64), G.CachedDecoder(c, 3, 64)
    close(dm.forward(tok[:, :33].contiguous().to(DEV), 0), dc.forward(tok[:, :33].contiguous(), 0), 3e-2, 3e-2, "prefill logits")
    for t in range(33, 40):
        got, want = dm.forward(tok[:, t:t + 1].contiguous().to(DEV), t), dc.forward(tok[:, t:t + 1].contiguous(), t)
    close(got, want, 3e-2, 3e-2, "decode logits")
    # the training forward pass of the same model agrees on the last position
    m.forward(tok.to(DEV))
    close(got, m.logits()[:, -1, :cfg.vocab_size], 3e-2, 3e-2, "decode vs training forward")
    prompts = [[5, 9, 11, 3], [7, 2], list(range(20, 50))]
    # bit-identical tokens need the same product kernel on both sides, so the weight-streaming product is switched off here
    d1, d2 = G.CachedDecoder(m, 3, 42), G.CachedDecoder(m, 3, 42)
    d1.skinny_rows = d2.skinny_rows = 0
    a = G.generate(m, prompts, max_gen_len=12, temperature=0.0, echo=True, decoder=d1)
    b = G.generate(m, prompts, max_gen_len=12, temperature=0.0, echo=True, use_kv=False, decoder=d2)
    assert a == b
    assert len(G.generate(m, prompts, max_gen_len=12, temperature=0.0)[0]) == 12          # default path: skinny product + graph
    for p, out in zip(prompts, a):
        assert out[:len(p)] == p and len(out) == len(p) + 12


def test_graph_replayed_decoding_step_equals_eager_and_refuses_positions_outside_the_cache():
    from llmc_b200 import _lib
    from llmc_b200.models import generate as G
    cfg = llama3.config_from_descriptor("llama3:l=2,c=256,h=4,kv=2,t=64,v=500,m=64,f=1.0")
    m = llama3.Llama(cfg, DEV, torch.bfloat16, recompute=1)
    m.init_random(5)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (2, 24), generator=g, dtype=torch.int32).to(DEV)
    eager, graphed = G.CachedDecoder(m, 2, 32), G.CachedDecoder(m, 2, 32)
    eager.forward(tok[:, :10].contiguous(), 0)
    graphed.forward(tok[:, :10].contiguous(), 0)
    gs = G.GraphStep(graphed, 2, 10)
    for t in range(10, 24):
        want = eager.forward(tok[:, t:t + 1].contiguous(), t)
        got = gs.step(tok[:, t:t + 1])
        assert torch.equal(got, want), "position %d" % t
    assert int(gs.pos.item()) == 24
    assert torch.equal(eager.kcache, graphed.kcache) and torch.equal(eager.vcache, graphed.vcache)
    # whole generations agree with and without the graph
    prompts = [[5, 9, 11, 3], [7, 2, 8]]
    assert G.generate(m, prompts, 20, temperature=0.0, use_graph=True) == G.generate(m, prompts, 20, temperature=0.0, use_graph=False)
    # a device position past the end of the cache: the kernels write nothing and say so in the status word
    _lib.read_status(clear=True)
    before = graphed.kcache.clone()
    gs.pos.fill_(32)
    gs.step(tok[:, :1])
    status = _lib.read_status(clear=True)
    assert status >> 24 == 3 and (status & 0xFFFFFF) in (0x30, 0x31), hex(status)
    assert torch.equal(graphed.kcache, before)


@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (4, 515, 264), (8, 500, 4096), (5, 128, 8), (3, 6144, 2048)])
def test_skinny_product(M, N, K):
    x, w = rnd(M, K), rnd(N, K, scale=0.05, seed=1)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    KN.matmul_skinny(out, x.to(DEV), w.to(DEV))
    ref = torch.empty(M, N)
    R.matmul_skinny(ref, x, w)
    close(out, ref, 2e-2, 1e-2, "matmul_skinny")
    # rows of a wider buffer (the decoder passes slices of padded buffers)
    big_x = torch.zeros(16, K + 8, dtype=torch.bfloat16, device=DEV)
    big_x[:M, :K] = x.to(DEV)
    out2 = torch.zeros(16, N + 3, dtype=torch.bfloat16, device=DEV)
    KN.matmul_skinny(out2[:M, :N], big_x[:M, :K], w.to(DEV))
    assert torch.equal(out2[:M, :N], out) and float(out2[M:].abs().sum()) == 0 and float(out2[:, N:].abs().sum()) == 0


def test_long_prompt_through_the_training_attention_kernel():
    """A prompt of 160 tokens per row takes the dense path (rotary + training attention kernel + cache copy); the same prompt
    through the per-query cache scan must give the same cache and logits up to bf16 rounding, and decoding continues from it."""
    from llmc_b200.models import generate as G
    cfg = llama3.config_from_descriptor("llama3:l=2,c=256,h=4,kv=2,t=256,v=500,m=64,f=1.0")
    m = llama3.Llama(cfg, DEV, torch.bfloat16, recompute=1)
    m.init_random(9)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (3, 170), generator=g, dtype=torch.int32).to(DEV)
    dense, scan = G.CachedDecoder(m, 3, 192), G.CachedDecoder(m, 3, 192)
    scan.dense_prefill_from = 10 ** 9
    ld, ls = dense.forward(tok[:, :160].contiguous(), 0), scan.forward(tok[:, :160].contiguous(), 0)
    assert dense._dense is not None and scan._dense is None
    assert torch.equal(dense.kcache[0], scan.kcache[0]) and torch.equal(dense.vcache[0], scan.vcache[0])   # same rotation arithmetic
    close(dense.kcache[1], scan.kcache[1], 3e-2, 3e-2, "keys of the second layer")
    close(ld, ls, 3e-2, 3e-2, "prefill logits, dense vs scan")
    for t in range(160, 170):
        ld, ls = dense.forward(tok[:, t:t + 1].contiguous(), t), scan.forward(tok[:, t:t + 1].contiguous(), t)
    close(ld, ls, 3e-2, 3e-2, "decode logits after dense prefill")


def test_trainer_samples_with_the_cache_during_training(tmp_path, capsys):
    """The training loop of a LLaMA model on the GPU with validation and sampling switched on: sampling goes through the cached
    decoder (graph-replayed steps) between optimizer steps and training continues afterwards."""
    import numpy as np
    from llmc_b200.train import TrainConfig, Trainer
    from llmc_b200.utils.dataloader import write_datafile
    rng = np.random.default_rng(0)
    write_datafile(str(tmp_path / "train.bin"), rng.integers(0, 70000, size=40000), "llama-3")
    write_datafile(str(tmp_path / "val.bin"), rng.integers(0, 70000, size=6000), "llama-3")
    c = TrainConfig(train_data_pattern=str(tmp_path / "train.bin"), val_data_pattern=str(tmp_path / "val.bin"),
                    load_filename="llama3:l=2,c=256,h=4,kv=2,t=128,v=70000,m=64,f=1.0", output_log_dir=str(tmp_path / "log"), B=2, T=128,
                    total_batch_size=256, learning_rate=1e-3, weight_decay=0.1, val_loss_every=2, val_max_steps=2, sample_every=2, genT=12,
                    max_steps=4, device="cuda", dtype="bf16", quiet=False, tokenizer_path=str(tmp_path / "none.bin"))
    t = Trainer(c)
    t.run()
    t.close()
    out = capsys.readouterr().out
    assert out.count("generating:") >= 2 and "val loss" in out
