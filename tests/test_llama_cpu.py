"""LLaMA-3 family on the CPU path: hand-written forward/backward against an autograd oracle, gradient accumulation,
a few optimizer steps, descriptors and the rotary table."""
import math

import pytest
import torch

from llmc_b200.models import llama3
from llmc_b200.parallel.dist import DistConfig
from llmc_b200.parallel.zero import ShardedAdamW
from oracle import llama_oracle_loss_and_grads

DESC = "llama3:l=2,c=64,h=4,kv=2,t=32,v=97,m=32,f=1.0"


def small_model(recompute=0, desc=DESC):
    m = llama3.Llama(llama3.config_from_descriptor(desc), "cpu", torch.float32, recompute=recompute)
    m.init_random(42)
    g = torch.Generator().manual_seed(1)
    for n in ("ln1w", "ln2w", "lnfw"):
        m.params[n].add_(torch.randn(m.params[n].shape, generator=g) * 0.1)
    for n in ("qkvw", "attprojw", "fc12w", "fcprojw"):                # larger weights so that every path carries signal
        m.params[n].mul_(4.0)
    return m


def batch(cfg, B=3, T=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


@pytest.mark.parametrize("recompute", [0, 1, 2])
@pytest.mark.parametrize("desc", [DESC, "llama3:l=2,c=64,h=4,kv=4,t=32,v=97,m=32,f=1.3", "llama3:l=1,c=64,h=4,kv=1,t=32,v=97,m=16,f=1.0"])
def test_forward_backward_matches_autograd(recompute, desc):
    m = small_model(recompute, desc)
    x, y = batch(m.cfg)
    ref_logits, ref_loss, ref_grads = llama_oracle_loss_and_grads(m, x, y)
    m.forward(x, y, write_dlogits=False)
    logits = m.logits()[..., :m.cfg.vocab_size]
    assert torch.allclose(logits, ref_logits[..., :m.cfg.vocab_size], atol=1e-4, rtol=1e-4)
    m.forward(x, y)
    m.backward()
    assert abs(float(m.loss()) - ref_loss) < 1e-4
    for name in llama3.PARAM_NAMES:
        got, want = m.grads[name], ref_grads[name]
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), "gradient of %s: max err %g" % (name, (got - want).abs().max())


def test_gradient_accumulation_equals_big_batch():
    m = small_model()
    x, y = batch(m.cfg, B=4)
    m.forward(x, y)
    m.backward()
    big = m.grads_flat.clone()
    big_loss = float(m.loss())
    for i in range(2):
        m.forward(x[2 * i:2 * i + 2], y[2 * i:2 * i + 2], grad_accum_steps=2, micro_step=i)
        m.backward(micro_step=i, last_micro_step=(i == 1))
    assert torch.allclose(m.grads_flat, big, atol=1e-5, rtol=1e-4)
    assert abs(float(m.loss(2)) - big_loss) < 1e-5


def test_overfit_single_batch_loss_decreases():
    m = small_model()
    x, y = batch(m.cfg)
    opt = ShardedAdamW(m, DistConfig(), zero_stage=0, use_master_weights=False, beta2=0.999)
    losses = []
    for step in range(10):
        m.forward(x, y)
        m.backward()
        losses.append(float(m.loss()))
        opt.grad_norm_sq()
        opt.step(1e-2, 0.0, step + 1)
    assert losses[-1] < losses[0] - 1.0, losses


def test_weight_decay_set_is_every_matrix():
    m = small_model()
    opt = ShardedAdamW(m, DistConfig(), zero_stage=0, use_master_weights=False)
    wd = {v["name"]: v["wd"] for v in opt.views(0.1)}
    assert all(wd[n] == pytest.approx(0.1) for n in llama3.DECAYED)
    assert all(wd[n] == 0.0 for n in ("ln1w", "ln2w", "lnfw"))


def test_descriptors():
    c = llama3.config_from_descriptor("llama3:8B")
    assert (c.num_layers, c.num_heads, c.num_kv_heads, c.channels, c.hidden_dim, c.head_size) == (32, 32, 8, 4096, 14336, 128)
    assert llama3.num_parameters(c) == 8030261248                    # the published parameter count of LLaMA-3.1 8B
    c = llama3.config_from_descriptor("llama3:70B")
    assert (c.hidden_dim, c.head_size) == (28672, 128)
    c = llama3.config_from_descriptor("llama3:405B")
    assert (c.hidden_dim, c.head_size, c.num_layers) == (53248, 128, 126)
    with pytest.raises(ValueError):
        llama3.config_from_descriptor("llama3:l=2,c=64,h=4,kv=3")
    with pytest.raises(ValueError):
        llama3.config_from_descriptor("llama3:q=1")


def test_rope_table_rescales_only_long_wavelengths():
    c = llama3.config_from_descriptor("llama3:8B")
    scaled = llama3.rope_table(c, 4)
    c.use_scaled_rope = False
    plain = llama3.rope_table(c, 4)
    ang_s = torch.atan2(scaled[1, :, 1], scaled[1, :, 0])
    ang_p = torch.atan2(plain[1, :, 1], plain[1, :, 0])
    assert torch.allclose(ang_s[:16], ang_p[:16])                      # short wavelengths untouched
    assert torch.allclose(ang_s[-1] * 8, ang_p[-1], rtol=1e-4)         # longest wavelength divided by the scale factor
    assert scaled.shape == (4, 64, 2) and float(scaled[0, :, 0].min()) == 1.0


# ---------------------------------------------------------------------------------------------------------------
# files and the trainer

import os

import numpy as np

from llmc_b200.train import TrainConfig, Trainer
from llmc_b200.utils import checkpoint, vislog
from llmc_b200.utils.dataloader import DataLoader, write_datafile

TDESC = "llama3:l=2,c=32,h=4,kv=2,t=16,v=70000,m=16,f=1.3"


def _files(tmp_path):
    rng = np.random.default_rng(0)
    # ids above 65535 force the 32-bit shard format of the LLaMA-3 tokenizer
    write_datafile(str(tmp_path / "train.bin"), rng.integers(0, 70000, size=4000), "llama-3")
    write_datafile(str(tmp_path / "val.bin"), rng.integers(0, 70000, size=600), "llama-3")


def _cfg(tmp_path, log, load=TDESC, **kw):
    return TrainConfig(train_data_pattern=str(tmp_path / "train.bin"), val_data_pattern=str(tmp_path / "val.bin"), load_filename=load,
                       output_log_dir=str(tmp_path / log), B=2, T=16, total_batch_size=64, learning_rate=1e-3, weight_decay=0.1,
                       val_loss_every=0, sample_every=0, device="cpu", dtype="fp32", quiet=True,
                       tokenizer_path=str(tmp_path / "none.bin"), **kw)


def test_wide_token_shards(tmp_path):
    toks = np.arange(100000, 100000 + 200, dtype=np.uint32)
    write_datafile(str(tmp_path / "w.bin"), toks, "llama-3")
    with open(tmp_path / "w.bin", "rb") as f:
        h = np.frombuffer(f.read(1024), dtype=np.int32)
    assert h[:3].tolist() == [20240801, 7, 200] and os.path.getsize(tmp_path / "w.bin") == 1024 + 4 * 200
    dl = DataLoader(str(tmp_path / "w.bin"), 2, 8, 1, 2, 0)
    x, y = dl.next_batch()
    assert x.flatten().tolist() == list(range(100016, 100032)) and y.flatten().tolist() == list(range(100017, 100033))
    dl.close()
    write_datafile(str(tmp_path / "n.bin"), np.arange(200), "gpt-2")
    with pytest.raises(Exception):
        DataLoader(str(tmp_path / "?.bin"), 2, 8, 0, 1, 0)              # 16-bit and 32-bit shards may not be mixed


def test_model_file_layout_and_roundtrip(tmp_path):
    cfg = llama3.config_from_descriptor(TDESC)
    m = llama3.Llama(cfg, "cpu", torch.float32)
    m.init_random(3)
    path = str(tmp_path / "llama.bin")
    checkpoint.write_model(path, m)
    assert checkpoint.model_family(path) == "llama3"
    with open(path, "rb") as f:
        h = np.frombuffer(f.read(1024), dtype=np.int32)
        body = np.frombuffer(f.read(), dtype=np.float32)
    assert h[:16].tolist() == [20240803, 3, 16, 70000, 2, 4, 2, 32, 1, 16, 0, 500000, 1, 4, 3, 1]
    H, C, L, V = cfg.hidden_dim, cfg.channels, cfg.num_layers, cfg.vocab_size
    qr = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size
    sizes = [V * C, L * C, L * qr * C, L * C * C, L * C, L * H * C, L * H * C, L * C * H, C, V * C]
    assert body.size == sum(sizes)                                        # the unpadded vocabulary, reference tensor order
    off = sum(sizes[:5])
    c_fc = torch.from_numpy(body[off:off + L * H * C].copy()).view(L, H, C)
    c_fc2 = torch.from_numpy(body[off + L * H * C:off + 2 * L * H * C].copy()).view(L, H, C)
    assert torch.equal(c_fc, m.params["fc12w"][:, :H]) and torch.equal(c_fc2, m.params["fc12w"][:, H:])
    hdr_cfg, version = checkpoint.read_model_header(path)
    assert hdr_cfg == cfg and version == 3
    m2 = llama3.Llama(cfg, "cpu", torch.float32)
    m2.params_flat.fill_(7.0)
    checkpoint.load_model(path, m2)
    assert torch.equal(m2.params_flat, m.params_flat)
    # a bf16 file loads into an fp32 model with the values rounded
    mb = llama3.Llama(cfg, "cpu", torch.bfloat16)
    mb.params_flat.copy_(m.params_flat)
    checkpoint.write_model(str(tmp_path / "b.bin"), mb)
    assert checkpoint.read_model_header(str(tmp_path / "b.bin"))[1] == 5
    checkpoint.load_model(str(tmp_path / "b.bin"), m2)
    assert torch.equal(m2.params_flat, mb.params_flat.float())


def test_trainer_runs_checkpoints_and_resumes_bit_exactly(tmp_path, capsys):
    _files(tmp_path)
    t = Trainer(_cfg(tmp_path, "runA", max_steps=6, checkpoint_every=3))
    assert t.model.family == "llama3"
    first = [t.train_step()["loss"] for _ in range(3)]
    t.write_checkpoint(3)
    rest = [t.train_step()["loss"] for _ in range(3)]
    final_a = t.model.params_flat.clone()
    t.close()
    assert first[0] > math.log(70000) - 0.5 and all(math.isfinite(x) for x in first + rest)
    t2 = Trainer(_cfg(tmp_path, "runA", max_steps=6, checkpoint_every=3, resume=1))
    assert t2.resuming and t2.step == 3 and t2.model.family == "llama3"
    rest2 = [t2.train_step()["loss"] for _ in range(3)]
    assert rest2 == rest and torch.equal(t2.model.params_flat, final_a)
    t2.close()
    # the whole loop with validation and sampling
    c = _cfg(tmp_path, "runB", max_steps=4)
    c.quiet, c.val_loss_every, c.val_max_steps, c.sample_every, c.genT = False, 2, 2, 4, 8
    t3 = Trainer(c)
    t3.run()
    t3.close()
    out = capsys.readouterr().out
    assert len(vislog.losses_from_stdout(out)) == 4 and "val loss" in out and "generating:" in out


def test_script_generates_from_prompt_tokens(tmp_path, capsys):
    """--inference_only of the LLaMA script: batched prompts given as token ids, with and without the key / value cache."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("train_llama3_script", os.path.join(os.path.dirname(__file__), "..", "train_llama3.py"))
    script = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(script)
    _files(tmp_path)
    common = ["--model", TDESC, "--input_bin", str(tmp_path / "train.bin"), "--input_val_bin", str(tmp_path / "val.bin"),
              "--batch_size", "2", "--sequence_length", "16", "--total_batch_size", "32", "--device", "cpu", "--dtype", "float32",
              "--inference_only", "1", "--prompt_tokens", "5,6,7;9", "--max_gen_len", "6", "--temperature", "0",
              "--tokenizer_path", str(tmp_path / "none.bin")]
    outs = []
    for kv in ("1", "0"):
        assert script.main(common + ["--use_kv", kv]) == 0
        lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("generated token ids:")]
        assert len(lines) == 2
        outs.append(lines)
    assert outs[0] == outs[1]
    assert all(len(l.split(":")[1].split()) == 6 for l in outs[0])


# ---------------------------------------------------------------------------------------------------------------
# against an independent implementation: Hugging Face's LlamaForCausalLM

@pytest.mark.parametrize("scaled", [False, True])
def test_logits_match_huggingface_llama_after_weight_conversion(scaled):
    transformers = pytest.importorskip("transformers")
    from llmc_b200.utils import llama_convert
    kw = dict(vocab_size=200, hidden_size=64, intermediate_size=192, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    if scaled:
        kw["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192}
    try:
        hf_cfg = transformers.LlamaConfig(**kw)
        torch.manual_seed(0)
        hf = transformers.LlamaForCausalLM(hf_cfg).float().eval()
    except Exception as e:            # a transformers release with a different configuration surface
        pytest.skip("cannot build the Hugging Face model: %s" % e)
    cfg = llama_convert.config_from_hf(hf_cfg)
    assert cfg.hidden_dim == 192 and cfg.use_scaled_rope == scaled and cfg.num_kv_heads == 2
    m = llama3.Llama(cfg, "cpu", torch.float32)
    llama_convert.from_hf_state_dict(m, hf.state_dict())
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, 200, (2, 32), generator=g)
    with torch.no_grad():
        want = hf(tok).logits
    m.forward(tok.to(torch.int32))
    got = m.logits()[..., :200]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()
    # and back: the exported state dict is the one we started from
    back = llama_convert.to_hf_state_dict(m)
    ref = hf.state_dict()
    for k, v in back.items():
        assert torch.equal(v, ref[k].float()), k


def test_export_to_huggingface_directory_and_back(tmp_path):
    transformers = pytest.importorskip("transformers")
    from llmc_b200.utils import export_hf, llama_convert
    cfg = llama3.config_from_descriptor("llama3:l=2,c=64,h=4,kv=2,t=64,v=200,m=32,f=1.0")
    m = llama3.Llama(cfg, "cpu", torch.float32)
    m.init_random(5)
    path = str(tmp_path / "m.bin")
    checkpoint.write_model(path, m)
    try:
        hf = export_hf.export(path, str(tmp_path / "hf"), "float32")
    except Exception as e:
        pytest.skip("cannot build the Hugging Face model: %s" % e)
    assert os.path.exists(tmp_path / "hf" / "config.json")
    tok = torch.randint(0, 200, (1, 16), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(tok).logits
    m.forward(tok.to(torch.int32))
    assert torch.allclose(m.logits()[..., :200], want, atol=2e-4, rtol=1e-3)
    # the converter CLI path: local directory -> model file -> identical parameters
    assert llama_convert.main(["--hf-dir", str(tmp_path / "hf"), "--out", str(tmp_path / "back.bin"), "--dtype", "float32"]) == 0
    m2 = llama3.Llama(checkpoint.read_model_header(str(tmp_path / "back.bin"))[0], "cpu", torch.float32)
    checkpoint.load_model(str(tmp_path / "back.bin"), m2)
    assert torch.equal(m2.params_flat, m.params_flat)
