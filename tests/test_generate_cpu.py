"""Generation with a key / value cache on the CPU path: cached logits against the training forward pass, batched prompts of
different lengths, stop tokens, echo, nucleus sampling (behaviour of LLaMA.generate / sample_top_p in the reference's
train_llama3.py:476-576)."""
import torch

from llmc_b200.models import generate as G
from llmc_b200.models import llama3

DESC = "llama3:l=2,c=64,h=4,kv=2,t=48,v=97,m=32,f=1.0"


def small_model(desc=DESC):
    m = llama3.Llama(llama3.config_from_descriptor(desc), "cpu", torch.float32, recompute=0)
    m.init_random(7)
    for n in ("qkvw", "attprojw", "fc12w", "fcprojw", "lmhead"):
        m.params[n].mul_(4.0)
    return m


def test_cached_logits_match_full_forward():
    m = small_model()
    g = torch.Generator().manual_seed(0)
    B, T = 3, 20
    tok = torch.randint(0, m.cfg.vocab_size, (B, T), generator=g, dtype=torch.int32)
    m.forward(tok)
    full = m.logits()[..., :m.cfg.vocab_size].clone()                 # (B, T, V)
    dec = G.CachedDecoder(m, B, 32)
    got = dec.forward(tok[:, :7].contiguous(), 0)                     # prefill of 7 tokens
    assert torch.allclose(got, full[:, 6], atol=1e-4, rtol=1e-4)
    got = dec.forward(tok[:, 7:10].contiguous(), 7)                   # three at once
    assert torch.allclose(got, full[:, 9], atol=1e-4, rtol=1e-4)
    for t in range(10, T):                                            # then one by one
        got = dec.forward(tok[:, t:t + 1].contiguous(), t)
        assert torch.allclose(got, full[:, t], atol=1e-4, rtol=1e-4), "position %d" % t


def test_dense_prefill_fills_the_cache_like_the_incremental_path():
    m = small_model()
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, m.cfg.vocab_size, (2, 24), generator=g, dtype=torch.int32)
    a, b = G.CachedDecoder(m, 2, 32), G.CachedDecoder(m, 2, 32)
    a.dense_prefill_from, b.dense_prefill_from = 8, 1000
    la, lb = a.forward(tok[:, :20].contiguous(), 0), b.forward(tok[:, :20].contiguous(), 0)
    assert torch.allclose(la, lb, atol=1e-5, rtol=1e-5)
    assert torch.allclose(a.kcache, b.kcache, atol=1e-6) and torch.allclose(a.vcache, b.vcache, atol=1e-6)
    for t in range(20, 24):
        la, lb = a.forward(tok[:, t:t + 1].contiguous(), t), b.forward(tok[:, t:t + 1].contiguous(), t)
    assert torch.allclose(la, lb, atol=1e-5, rtol=1e-5)


def test_single_kv_head_and_full_heads():
    for desc in ("llama3:l=1,c=64,h=4,kv=1,t=32,v=50,m=16,f=1.0", "llama3:l=1,c=64,h=4,kv=4,t=32,v=50,m=16,f=1.3"):
        m = small_model(desc)
        tok = torch.arange(24, dtype=torch.int32).view(2, 12) % m.cfg.vocab_size
        m.forward(tok)
        full = m.logits()[..., :m.cfg.vocab_size].clone()
        dec = G.CachedDecoder(m, 2, 16)
        dec.forward(tok[:, :5].contiguous(), 0)
        for t in range(5, 12):
            got = dec.forward(tok[:, t:t + 1].contiguous(), t)
        assert torch.allclose(got, full[:, 11], atol=1e-4, rtol=1e-4)


def test_generate_cache_equals_recompute_and_forces_prompts():
    m = small_model()
    prompts = [[5, 9, 11, 3], [7, 2], [1, 2, 3, 4, 5, 6, 8]]
    with_cache = G.generate(m, prompts, max_gen_len=10, temperature=0.0, echo=True)
    without = G.generate(m, prompts, max_gen_len=10, temperature=0.0, echo=True, use_kv=False)
    assert with_cache == without
    for p, out in zip(prompts, with_cache):
        assert out[:len(p)] == p
        assert len(out) <= len(p) + 10
    # every row continues as it would alone: batching must not leak between rows
    for p, out in zip(prompts, with_cache):
        alone = G.generate(m, [p], max_gen_len=10, temperature=0.0, echo=True)[0]
        n = min(len(alone), len(out))
        assert alone[:n] == out[:n]
    no_echo = G.generate(m, prompts, max_gen_len=10, temperature=0.0)
    for p, full, tail in zip(prompts, with_cache, no_echo):
        assert full[len(p):] == tail


def test_stop_tokens_cut_the_output_and_end_the_loop():
    m = small_model()
    prompts = [[5, 9, 11, 3], [7, 2]]
    free = G.generate(m, prompts, max_gen_len=12, temperature=0.0)
    stop = free[0][2]                                                  # a token the first row is known to produce
    cut = G.generate(m, prompts, max_gen_len=12, temperature=0.0, stop_tokens=(stop,))
    assert cut[0] == free[0][:free[0].index(stop)]
    assert stop not in cut[1]
    assert free[1][:len(cut[1])] == cut[1]


def test_context_window_bounds_generation():
    m = small_model()
    out = G.generate(m, [list(range(1, 41))], max_gen_len=100, temperature=0.0, echo=True)[0]
    assert len(out) == m.cfg.max_seq_len


def test_sample_top_p():
    g = torch.Generator().manual_seed(0)
    probs = torch.tensor([[0.5, 0.3, 0.15, 0.05]]).repeat(4000, 1)
    picks = G.sample_top_p(probs, 0.7, g)                              # nucleus = {0, 1}: mass before token 2 is 0.8 > 0.7
    counts = torch.bincount(picks, minlength=4).float() / 4000
    assert counts[2] == 0 and counts[3] == 0
    assert abs(counts[0] - 0.625) < 0.03 and abs(counts[1] - 0.375) < 0.03
    assert torch.equal(G.sample_top_p(probs[:8], 0.0, g), torch.zeros(8, dtype=torch.int64))   # only the top token survives
    g1, g2 = torch.Generator().manual_seed(3), torch.Generator().manual_seed(3)
    m = small_model()
    a = G.generate(m, [[4, 5, 6]], 8, temperature=0.8, top_p=0.9, generator=g1)
    b = G.generate(m, [[4, 5, 6]], 8, temperature=0.8, top_p=0.9, generator=g2)
    assert a == b
