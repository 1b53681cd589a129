"""Host runtime: RNG parity with PyTorch, data loaders (the cases of the reference's dev/test/test_dataloader.c),
evaluation loader, tokenizer, sampler, schedules, outlier detector (dev/test/test_outlier_detector.c), logger,
checkpoint files, command line."""
import math
import os
import struct

import numpy as np
import pytest
import torch

from llmc_b200.models import gpt2
from llmc_b200.train import TrainConfig, Trainer, UsageError, parse_args
from llmc_b200.utils import checkpoint, mfu, vislog
from llmc_b200.utils.dataloader import DataLoader, EvalLoader, write_datafile, write_evalfile
from llmc_b200.utils.logger import Logger
from llmc_b200.utils.outlier import OutlierDetector
from llmc_b200.utils.rand import MT19937
from llmc_b200.utils.sampler import Sampler
from llmc_b200.utils.schedulers import LearningRateScheduler
from llmc_b200.utils.tokenizer import Tokenizer, printable, write_tokenizer


def test_mt19937_matches_torch_streams():
    r, g = MT19937(42), torch.Generator().manual_seed(42)
    assert torch.equal(r.uniform(1000), torch.empty(1000).uniform_(generator=g))
    a, t = r.normal(1000, 0.0, 0.02), torch.empty(1000).normal_(0.0, 0.02, generator=g)
    assert torch.allclose(a, t, atol=1e-7)
    a, t = r.normal(37, 1.0, 2.0), torch.empty(37).normal_(1.0, 2.0, generator=g)      # ragged tail path
    assert torch.allclose(a, t, atol=1e-6)
    a, t = r.normal(7, 0.0, 1.0), torch.empty(7).normal_(0.0, 1.0, generator=g)        # fewer than 16: double path
    assert torch.allclose(a, t, atol=1e-6)
    # raw 32-bit stream equals numpy's MT19937 seeded the same way
    r2 = MT19937(1234)
    ref = np.random.RandomState(1234)
    assert [r2.randint32() for _ in range(5)] == [int(x) for x in ref.randint(0, 2 ** 32, size=5, dtype=np.uint64)]
    # state round trip
    st = r.get_state()
    x = r.randint32()
    r.set_state(st)
    assert len(st) == 2520 and r.randint32() == x
    p = r.permutation(100)
    assert sorted(p.tolist()) == list(range(100))


def _shards(tmp_path, n=4, ntok=140):
    for i in range(n):
        write_datafile(str(tmp_path / ("shard_%04d.bin" % i)), np.arange(i * ntok, (i + 1) * ntok, dtype=np.uint16))
    return str(tmp_path / "shard_*.bin")


def test_dataloader_simple_and_multiprocess(tmp_path):
    pat = _shards(tmp_path)
    B, T = 4, 8
    dl = DataLoader(pat, B, T, 0, 1, False)
    assert dl.num_tokens == 4 * 140 and dl.num_shards == 4
    per_shard = (140 - 1) // (B * T)
    expect = 0
    for epoch_batch in range(2 * 4 * per_shard):
        shard, idx = (epoch_batch // per_shard) % 4, epoch_batch % per_shard
        x, y = dl.next_batch()
        start = shard * 140 + idx * B * T
        assert x.flatten().tolist() == list(range(start, start + B * T))
        assert y.flatten().tolist() == list(range(start + 1, start + B * T + 1))
    # two processes read interleaved slots of every global batch
    l0, l1 = DataLoader(pat, B, T, 0, 2, False), DataLoader(pat, B, T, 1, 2, False)
    x0, _ = l0.next_batch()
    x1, _ = l1.next_batch()
    assert x0.flatten().tolist() == list(range(0, 32)) and x1.flatten().tolist() == list(range(32, 64))
    for l in (dl, l0, l1):
        l.close()


def test_dataloader_shuffle_covers_everything_and_resumes(tmp_path):
    pat = _shards(tmp_path)
    B, T = 4, 8
    per_shard = (140 - 1) // (B * T)
    dl = DataLoader(pat, B, T, 0, 1, True, prefetch=True)
    counts = np.zeros(4 * 140, dtype=np.int64)
    order = []
    for _ in range(4 * per_shard):
        x, _ = dl.next_batch()
        counts[x.flatten().numpy()] += 1
        order.append(int(x[0, 0]))
    # every in-range window is visited exactly once per epoch, in a shuffled order
    assert set(counts.tolist()) <= {0, 1} and counts.sum() == 4 * per_shard * B * T
    assert order != sorted(order)
    # save the position mid-epoch, keep going, then restore into a fresh loader: the continuation must be identical
    shard_idx, sample_idx = dl.position()
    si, ii, raw = dl.shuffle_state()
    nxt = [dl.next_batch()[0].clone() for _ in range(5)]
    d2 = DataLoader(pat, B, T, 0, 1, True)
    d2.set_shuffle_state(si, ii, raw)
    d2.resume(shard_idx, sample_idx)
    for want in nxt:
        assert torch.equal(d2.next_batch()[0], want)
    dl.close(); d2.close()


def test_dataloader_rejects_bad_files(tmp_path):
    bad = tmp_path / "bad.bin"
    bad.write_bytes(struct.pack("<256i", *([1] + [0] * 255)))
    with pytest.raises(RuntimeError, match="bad magic"):
        DataLoader(str(bad), 1, 4)
    with pytest.raises(RuntimeError, match="no files"):
        DataLoader(str(tmp_path / "nothing_*.bin"), 1, 4)


def test_evalloader(tmp_path):
    exs = []
    for i in range(5):
        exs.append(dict(ctx=[10 + i, 11, 12], endings=[[20], [21, 22], [23], [24, 25, 26]], label=i % 4))
    path = str(tmp_path / "eval.bin")
    write_evalfile(path, exs)
    B, T = 8, 16
    el = EvalLoader(path, B, T)
    assert el.num_examples == 5 and el.num_batches == 3
    x, y, mask = el.next_batch()
    assert x[0, :4].tolist() == [10, 11, 12, 20] and x[1, :5].tolist() == [10, 11, 12, 21, 22]
    assert y[1, 2:4].tolist() == [21, 22] and mask[1].tolist()[:5] == [0, 0, 1, 1, 0]
    # losses that make completion `label` the cheapest -> all examples of the batch counted correct
    losses = torch.full((B, T), 5.0)
    for e in range(2):
        losses[e * 4 + exs[e]["label"]] = 0.1
    assert el.stat_losses(losses) == 2
    el.close()


def test_tokenizer_sampler(tmp_path):
    path = str(tmp_path / "tok.bin")
    write_tokenizer(path, [b"a", b" the", b"\x01", b"<|endoftext|>"], eot=3)
    tk = Tokenizer(path)
    assert tk.init_ok and tk.vocab_size == 4 and tk.eot_token == 3
    assert tk.decode(1) == b" the" and printable(tk.decode(2)) == "" and tk.decode(9) is None
    assert not Tokenizer(str(tmp_path / "missing.bin")).init_ok
    s = Sampler(1337)
    a = [s.random_u32() for _ in range(3)]
    s2 = Sampler(1337)
    assert a == [s2.random_u32() for _ in range(3)] and 0.0 <= s.random_f32() < 1.0
    logits = torch.tensor([0.0, 10.0, 0.0])
    assert s.sample_softmax(logits, 0.5) == 1 and s.sample_softmax(logits, 0.0) == 0


def test_schedulers():
    c = LearningRateScheduler("cosine", 1.0, 10, 110, 0.1)
    assert c.get_learning_rate(0) == pytest.approx(0.1) and c.get_learning_rate(9) == pytest.approx(1.0)
    assert c.get_learning_rate(60) == pytest.approx(0.1 + 0.5 * 0.9) and c.get_learning_rate(110) == pytest.approx(0.1)
    l = LearningRateScheduler("linear", 1.0, 0, 100, 0.0)
    assert l.get_learning_rate(50) == pytest.approx(0.5)
    assert LearningRateScheduler("constant", 0.3, 5, 100, 0.0).get_learning_rate(77) == pytest.approx(0.3)
    w = LearningRateScheduler("wsd", 1.0, 10, 100, 0.0)
    assert w.get_learning_rate(50) == 1.0 and w.get_learning_rate(90) == pytest.approx(1.0 - math.sqrt(0.5))
    with pytest.raises(ValueError):
        LearningRateScheduler("nope", 1.0, 0, 1, 0.0)


def test_outlier_detector():
    d = OutlierDetector()
    g = torch.Generator().manual_seed(0)
    for i in range(OutlierDetector.WINDOW):
        assert math.isnan(d.update(float(torch.randn(1, generator=g))))
    for i in range(OutlierDetector.WINDOW):
        assert abs(d.update(float(torch.randn(1, generator=g)))) < 4.0
    assert d.update(10.0) > 5.0


def test_logger_and_vislog(tmp_path):
    lg = Logger(str(tmp_path), 0)
    lg.log_val(0, 3.5); lg.log_train(0, 3.4, 1e-4, 1.25); lg.log_eval(10, 0.29)
    s = vislog.parse_logfile(str(tmp_path / "main.log"))
    assert s["tel"][0] == 3.5 and s["trl"][0] == 3.4 and s["eval"][10] == 0.29 and s["norm"][0] == 1.25
    assert not Logger(str(tmp_path / "r1"), 1).active
    txt = "step    1/10 | loss 5.270009 (+nanz)| norm 1.0 (+nanz)| lr 1e-4 | 10.0 ms | 1.0% bf16 MFU | 10 tok/s\n"
    assert vislog.losses_from_stdout(txt) == [5.270009]
    assert vislog.check_losses([5.27], [5.270009]) and not vislog.check_losses([6.0], [5.27])


def test_mfu_table_knows_blackwell():
    assert mfu.get_flops_promised("NVIDIA B200") == 2250.0 and mfu.get_flops_promised("Mystery GPU") == -1.0
    assert mfu.estimate_mfu(803.5e6, 65536, 0.0765, "NVIDIA B200") == pytest.approx(803.5e6 * 65536 / 0.0765 / 2.25e15)

    class FakeNVML:            # telemetry is read-only and tested against a fake
        NVML_CLOCK_SM, NVML_TEMPERATURE_GPU = 1, 0
        def nvmlInit(self): pass
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetUtilizationRates(self, h): return type("U", (), dict(gpu=97, memory=40))()
        def nvmlDeviceGetClockInfo(self, h, k): return 1600
        def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
        def nvmlDeviceGetPowerUsage(self, h): return 950000
        def nvmlDeviceGetEnforcedPowerLimit(self, h): return 1000000
        def nvmlDeviceGetTemperature(self, h, k): return 60
        def nvmlDeviceGetCurrentClocksThrottleReasons(self, h): return 4
    info = mfu.GPUTelemetry(3, FakeNVML()).read()
    assert info["clock"] == 1600 and info["power"] == 950.0 and "1600/1965" in mfu.GPUTelemetry.format(info)


def test_cli_parser():
    c = parse_args("-e d12 -b 64 -t 1024 -d 524288 -z 1 -lg 5 -ge 2 -pi fs -pf /tmp/x -sl 7.0 -nk 5".split())
    assert (c.load_filename, c.B, c.T, c.total_batch_size, c.zero_stage, c.log_gpu_every, c.gelu_fusion) == ("d12", 64, 1024, 524288, 1, 5, 2)
    assert c.nccl_init_method == "fs" and c.fs_path == "/tmp/x" and c.skip_update_lossz == 7.0 and c.checkpoints_keep == 5
    assert parse_args(["-pm", "tcp"]).nccl_init_method == "tcp"          # alias printed by the reference's usage text
    for bad in (["-b"], ["-zz", "1"], ["-b", "x"]):
        with pytest.raises(UsageError):
            parse_args(bad)


def _tiny_files(tmp_path):
    rng = np.random.default_rng(0)
    write_datafile(str(tmp_path / "train.bin"), rng.integers(0, 97, size=4000, dtype=np.uint16))
    write_datafile(str(tmp_path / "val.bin"), rng.integers(0, 97, size=600, dtype=np.uint16))
    cfg = gpt2.GPTConfig(max_seq_len=16, vocab_size=97, padded_vocab_size=104, num_layers=2, num_heads=2, channels=32)
    m = gpt2.GPT(cfg, "cpu", torch.float32)
    m.init_random(42)
    checkpoint.write_model(str(tmp_path / "init.bin"), m)
    return cfg


def _train_cfg(tmp_path, log, **kw):
    return TrainConfig(train_data_pattern=str(tmp_path / "train.bin"), val_data_pattern=str(tmp_path / "val.bin"),
                       load_filename=str(tmp_path / "init.bin"), output_log_dir=str(tmp_path / log), B=2, T=16, total_batch_size=64,
                       learning_rate=1e-3, weight_decay=0.1, val_loss_every=0, sample_every=0, device="cpu", dtype="fp32", quiet=True,
                       tokenizer_path=str(tmp_path / "none.bin"), **kw)


def test_checkpoint_files_and_bit_exact_resume(tmp_path):
    """The scheme of the reference's test_gpt2.cu:326-367: checkpoint, continue, reload, continue again -> identical."""
    cfg = _tiny_files(tmp_path)
    hdr_cfg, version = checkpoint.read_model_header(str(tmp_path / "init.bin"))
    assert hdr_cfg == cfg and version == 3
    with open(tmp_path / "init.bin", "rb") as f:
        h = np.frombuffer(f.read(1024), dtype=np.int32)
    assert h[:8].tolist() == [20240326, 3, 16, 97, 2, 2, 32, 104]
    assert os.path.getsize(tmp_path / "init.bin") == 1024 + 4 * gpt2.num_parameters(cfg)

    t = Trainer(_train_cfg(tmp_path, "runA", max_steps=6, checkpoint_every=3))
    first = [t.train_step()["loss"] for _ in range(3)]
    t.write_checkpoint(3)
    rest = [t.train_step()["loss"] for _ in range(3)]
    final_a = t.model.params_flat.clone()
    t.close()
    assert checkpoint.find_max_step(str(tmp_path / "runA")) == 3
    with open(tmp_path / "runA" / "state_00000003_00000.bin", "rb") as f:
        sh = np.frombuffer(f.read(1024), dtype=np.int32)
    assert sh[0] == 20240527 and sh[1] == 1 and sh[2] == 1 and sh[3] == 0 and sh[10] == 3 and sh[5] == 1

    t2 = Trainer(_train_cfg(tmp_path, "runA", max_steps=6, checkpoint_every=3, resume=1))
    assert t2.resuming and t2.step == 3
    rest2 = [t2.train_step()["loss"] for _ in range(3)]
    assert rest2 == rest and torch.equal(t2.model.params_flat, final_a)
    t2.close()
    assert all(math.isfinite(x) for x in first + rest)
    checkpoint.delete_checkpoint(str(tmp_path / "runA"), 3, 0)
    assert checkpoint.find_max_step(str(tmp_path / "runA")) == -1


def test_training_loop_end_to_end(tmp_path, capsys):
    _tiny_files(tmp_path)
    c = _train_cfg(tmp_path, "runB", max_steps=4, checkpoint_every=2, checkpoints_keep=1)
    c.quiet, c.val_loss_every, c.val_max_steps, c.sample_every, c.genT = False, 2, 2, 4, 8
    t = Trainer(c)
    t.run()
    t.close()
    out = capsys.readouterr().out
    losses = vislog.losses_from_stdout(out)
    assert len(losses) == 4 and "val loss" in out and "generating:" in out
    log = vislog.parse_logfile(str(tmp_path / "runB" / "main.log"))
    assert sorted(log["trl"]) == [0, 1, 2, 3] and 4 in log["tel"]
    assert os.path.exists(tmp_path / "runB" / "DONE_00000004") and not os.path.exists(tmp_path / "runB" / "model_00000002.bin")


def test_cpu_matmul_kernels_match_torch():
    """The two CPU matmuls of the host library (plain and register-tiled), odd sizes and thread counts included."""
    from llmc_b200 import bench_cpu_matmul as bm
    g = torch.Generator().manual_seed(0)
    for BT, C, OC, threads in ((13, 24, 17, 1), (64, 48, 40, 3), (9, 8, 8, 4)):
        inp, w, b = torch.randn(BT, C, generator=g), torch.randn(OC, C, generator=g), torch.randn(OC, generator=g)
        ref = inp @ w.t() + b
        for kind in ("naive", "tiled"):
            assert torch.allclose(bm.matmul(kind, inp, w, b, threads), ref, atol=1e-4, rtol=1e-4), (kind, BT, C, OC)
        assert torch.allclose(bm.matmul("tiled", inp, w, None, threads), inp @ w.t(), atol=1e-4, rtol=1e-4)
