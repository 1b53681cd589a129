"""The GPT-2 debug-state file (magic 20240327, version 2): written from the autograd oracle, read back, and used the way the
reference's test_gpt2.c uses its copy: logits, loss and all 16 gradient tensors of the model under test against the file."""
import numpy as np
import pytest
import torch

from llmc_b200.models import gpt2
from llmc_b200.utils import debug_state
from oracle import oracle_loss_and_grads
from test_model_cpu import batch, small_model


def test_round_trip_and_model_check(tmp_path):
    m = small_model()
    x, y = batch(m.cfg)
    logits, loss, grads = oracle_loss_and_grads(m, x, y)
    path = str(tmp_path / "debug_state.bin")
    debug_state.write_debug_state(path, m.cfg, x, y, logits, loss, grads)
    B, T = x.shape
    V, Vp, C = m.cfg.vocab_size, m.cfg.padded_vocab_size, m.cfg.channels
    # byte layout of the reference: header, x, y, logits over the unpadded vocabulary, loss, gradients with a padded embedding
    expected = 1024 + 2 * 4 * B * T + 4 * B * T * V + 4 + 4 * m.num_parameters
    import os
    assert os.path.getsize(path) == expected
    head = np.fromfile(path, dtype=np.int32, count=4)
    assert list(head) == [20240327, 2, B, T]
    st = debug_state.read_debug_state(path, m.cfg)
    assert torch.equal(st["x"], x) and torch.equal(st["y"], y)
    assert torch.equal(st["logits"], logits[..., :V])
    assert st["grads"]["wte"].shape == (Vp, C) and float(st["grads"]["wte"][V:].abs().max()) == 0.0
    dev = debug_state.check_model(m, st)
    assert dev["logits"] < 1e-4 and dev["loss"] < 1e-4
    for name, d in dev["grads"].items():
        assert d < 2e-3, (name, d)


def test_from_model_and_rejections(tmp_path):
    m = small_model()
    x, y = batch(m.cfg, B=2, T=8, seed=3)
    path = str(tmp_path / "own.bin")
    debug_state.from_model(path, m, x, y)
    st = debug_state.read_debug_state(path, m.cfg)
    dev = debug_state.check_model(m, st)
    assert dev["logits"] == 0.0 and dev["loss"] == 0.0 and max(dev["grads"].values()) == 0.0
    raw = bytearray(open(path, "rb").read())
    bad = str(tmp_path / "bad.bin")
    open(bad, "wb").write(bytes(raw[:-8]))
    with pytest.raises(IOError):
        debug_state.read_debug_state(bad, m.cfg)
    raw[0:4] = np.int32(1234).tobytes()
    open(bad, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        debug_state.read_debug_state(bad, m.cfg)
