"""Checkpoint -> resume on GPUs through real files (the scheme of the reference's test_gpt2.cu:326-367): train 10 steps, write
model and state files, train 10 more; start again from the files, train the same 10: losses and parameters must be identical
bit for bit.  This exercises the replay of the stochastic-rounding seeds, the re-rounding of bf16 parameters from the fp32 master
copy and the data loader's state, on one GPU and under ZeRO-1 on the in-kernel NVLink backend (2 GPUs)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from llmc_b200.models import gpt2
from llmc_b200.utils import checkpoint, debug_state
from llmc_b200.utils.dataloader import write_datafile

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "resume_worker.py")


def files(tmp_path):
    rng = np.random.default_rng(0)
    write_datafile(str(tmp_path / "train.bin"), rng.integers(0, 1000, size=200000, dtype=np.uint16))
    cfg = gpt2.GPTConfig(max_seq_len=128, vocab_size=1000, padded_vocab_size=1024, num_layers=2, num_heads=2, channels=128)
    m = gpt2.GPT(cfg, "cpu", torch.float32)
    m.init_random(42)
    checkpoint.write_model(str(tmp_path / "init.bin"), m)
    return cfg


def run(world, args, port):
    if world == 1:
        cmd = [sys.executable, WORKER] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
               "--master-port", str(port), WORKER] + args
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.parametrize("world,backend", [(1, "single"), (2, "p2p"), (2, "nccl")])
def test_resume_is_bit_identical(tmp_path, world, backend):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    files(tmp_path)
    full, resumed = str(tmp_path / "full.json"), str(tmp_path / "resumed.json")
    common = ["--dir", str(tmp_path), "--run-name", "run", "--backend", backend]
    run(world, common + ["--steps", "20", "--checkpoint-at", "10", "--out", full], 29581)
    assert os.path.exists(tmp_path / "run" / "DONE_00000010")
    for r in range(world):
        assert os.path.exists(tmp_path / "run" / ("state_00000010_%05d.bin" % r))
    run(world, common + ["--steps", "20", "--resume", "1", "--out", resumed], 29582)
    a, b = json.load(open(full)), json.load(open(resumed))
    assert b["start"] == 10 and len(b["losses"]) == 10
    if world > 1:
        assert a["backend"] == backend
    assert a["losses"][10:] == b["losses"], (a["losses"][10:], b["losses"])
    assert a["params"] == b["params"]


def test_bf16_model_against_debug_state_file(tmp_path):
    """The reference's test_gpt2.cu scheme: a debug-state file written from the fp32 CPU path, checked by the bf16 kernel path
    with its tolerances (logits within bf16 resolution of their magnitude, loss 5e-2, gradients per tensor)."""
    cfg = gpt2.GPTConfig(max_seq_len=128, vocab_size=1000, padded_vocab_size=1024, num_layers=2, num_heads=2, channels=128)
    cm = gpt2.GPT(cfg, "cpu", torch.float32, recompute=0)
    cm.init_random(42)
    g = torch.Generator().manual_seed(4)
    tok = torch.randint(0, cfg.vocab_size, (4, 129), generator=g, dtype=torch.int32)
    path = str(tmp_path / "debug_state.bin")
    debug_state.from_model(path, cm, tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
    gm = gpt2.GPT(cfg, "cuda", torch.bfloat16, recompute=0)
    gm.params_flat.copy_(cm.params_flat)
    dev = debug_state.check_model(gm, debug_state.read_debug_state(path, cfg))
    assert dev["logits"] < 5e-2 and dev["loss"] < 5e-2, dev
    st = debug_state.read_debug_state(path, cfg)
    for name, d in dev["grads"].items():
        scale = float(st["grads"][name].abs().max())
        assert d < 3e-2 * max(scale, 1e-2) + 2e-3, (name, d, scale)
