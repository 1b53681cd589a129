"""Runs in a child process with LLMC_DEBUG_CHECKS=1 (see test_debug_build_gpu.py): the kernels of the debug library must train
a tiny model with a clean status word, and must REPORT -- not fault on -- an id outside the embedding table and a misaligned
16-byte access.  Prints one JSON line."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from llmc_b200 import _lib
from llmc_b200.models import gpt2
from llmc_b200.ops import kernels as K
from llmc_b200.parallel.dist import DistConfig
from llmc_b200.parallel.zero import ShardedAdamW


def main():
    out = {"debug_lib": int(_lib.cuda().llmc_debug_checks_enabled())}
    if out["debug_lib"] != 1:
        print(json.dumps(out))
        return 1                      # never run the cases below on the normal library: it has no checks to catch them
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = gpt2.GPTConfig(max_seq_len=64, vocab_size=1000, padded_vocab_size=1024, num_layers=2, num_heads=2, channels=128)
    model = gpt2.GPT(cfg, dev, torch.bfloat16, recompute=0)
    model.init_random(42)
    opt = ShardedAdamW(model, DistConfig(0, 1, 0, dev), 0, True)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, 65), generator=g, dtype=torch.int32)
    x, y = tok[:, :-1].contiguous().to(dev), tok[:, 1:].contiguous().to(dev)
    losses = []
    for step in range(3):
        model.forward(x, y)
        model.backward()
        losses.append(float(model.loss().item()))
        opt.grad_norm_sq()
        opt.step(1e-3, 0.0, step + 1)
    out["losses"] = losses
    out["status_after_training"] = _lib.read_status()
    # an id outside the table: reported, clamped, nothing faults
    C, V = 128, 1000
    wte = torch.randn(V, C, device=dev).bfloat16()
    wpe = torch.randn(64, C, device=dev).bfloat16()
    bad = x.clone()
    bad[0, 0] = V + 5
    emb = torch.empty(4, 64, C, device=dev, dtype=torch.bfloat16)
    K.encoder_forward(emb, bad, wte, wpe)
    out["status_bad_token"] = _lib.read_status()
    out["bad_token_output_finite"] = bool(torch.isfinite(emb.float()).all())
    # a misaligned 16-byte access: reported, skipped
    buf = torch.zeros(1024 + 8, device=dev, dtype=torch.bfloat16)
    dst = torch.empty(1024, device=dev, dtype=torch.bfloat16)
    K.gelu_forward(dst, buf[1:1025])
    out["status_misaligned"] = _lib.read_status()
    # the context is still usable and the status is clean again
    K.gelu_forward(dst, buf[:1024])
    torch.cuda.synchronize()
    out["status_after"] = _lib.read_status()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
