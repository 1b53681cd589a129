"""CI loss check: trains a small random-init GPT-2 for ten steps on the GPU (bf16 kernels) and on the CPU (fp32 restatement) from
the same parameters and token stream, and fails if a GPU loss leaves a 5 % band around the CPU loss of the same step
(reference: dev/loss_checker_ci.py, which compares the trainer's stdout with stored fp32 losses).

    python -m llmc_b200.utils.ci_loss_check [--steps 10] [--layers 4]
"""
import argparse
import sys

import torch

from ..models import gpt2
from ..parallel.dist import DistConfig
from ..parallel.zero import ShardedAdamW
from .vislog import check_losses


def run(device, dtype, steps, layers, B=4, T=256):
    cfg = gpt2.GPTConfig(max_seq_len=T, vocab_size=50257, padded_vocab_size=50304, num_layers=layers, num_heads=12, channels=768)
    m = gpt2.GPT(cfg, device, dtype, recompute=1)
    m.init_random(42)
    opt = ShardedAdamW(m, DistConfig(0, 1, 0, torch.device(device)), 0, True)
    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)     # one batch, overfitted: losses must fall
    x, y = tok[:, :-1].contiguous().to(device), tok[:, 1:].contiguous().to(device)
    losses = []
    for step in range(steps):
        m.forward(x, y)
        m.backward()
        opt.grad_norm_sq()
        opt.step(1e-4, 0.0, step + 1)
        losses.append(float(m.loss()))
    return losses


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--layers", type=int, default=4)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("no CUDA device: nothing to check")
        return 0
    want = run("cpu", torch.float32, a.steps, a.layers)
    got = run("cuda", torch.bfloat16, a.steps, a.layers)
    for s, (w, g) in enumerate(zip(want, got)):
        print("step %2d  cpu fp32 %.4f  gpu bf16 %.4f" % (s, w, g))
    if not check_losses(got, want, rel_tol=0.05) or not got[-1] < got[0]:
        print("LOSS MISMATCH")
        return 1
    print("LOSS OK")
    return 0


if __name__ == "__main__":
    sys.exit(main())
