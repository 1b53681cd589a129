"""Worker for the multi-process tests: trains a small GPT for a few steps under data parallelism / ZeRO-1 and lets rank 0
write the resulting parameters and loss curve.  Launched by torch.distributed.run (gloo on CPU, NCCL on GPUs), or run
directly with --world 1 --accum N to produce the single-process result the parallel runs must match."""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from llmc_b200.models import gpt2, llama3  # noqa: E402
from llmc_b200.parallel import dist as pdist  # noqa: E402
from llmc_b200.parallel.zero import ShardedAdamW  # noqa: E402


def batch_for(step, slot, B, T, V):
    g = torch.Generator().manual_seed(1000 * step + slot)
    tok = torch.randint(0, V, (B, T + 1), generator=g, dtype=torch.int32)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--backend", default="nccl")       # nccl (gloo on CPU) | p2p
    ap.add_argument("--zero", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--slots", type=int, default=2)    # data-parallel slots per optimizer step (= world size of the parallel run)
    ap.add_argument("--out", required=True)
    ap.add_argument("--family", default="gpt2")        # gpt2 | llama3
    ap.add_argument("--fail-rank", type=int, default=-1)   # this rank raises before its second step (failure-detection test)
    ap.add_argument("--skip-step", type=int, default=-1)   # every rank skips the update of this step (as the outlier detector would)
    a = ap.parse_args()

    d = pdist.init_distributed(device_type=a.device, timeout_s=20 if a.fail_rank >= 0 else 120)
    world, rank = d.num_processes, d.process_rank
    dtype = torch.bfloat16 if a.device == "cuda" else torch.float32
    cfg = gpt2.GPTConfig(max_seq_len=64, vocab_size=512, padded_vocab_size=512, num_layers=2, num_heads=2, channels=128)
    arena, bufs, allocator = None, {}, None
    if world > 1 and a.backend == "p2p":
        from llmc_b200.parallel import p2p
        arena = p2p.try_create(None, d, a.zero, print)
        assert arena is not None, "symmetric memory unavailable"

        def allocator(kind, numel, dt):
            bufs[kind] = arena.alloc(numel, dt)
            return bufs[kind][0]
    if a.family == "llama3":
        cfg = llama3.config_from_descriptor("llama3:l=2,c=128,h=2,kv=1,t=64,v=512,m=64,f=1.0")
        model = llama3.Llama(cfg, d.device, dtype, recompute=0, flat_allocator=allocator)
    else:
        model = gpt2.GPT(cfg, d.device, dtype, recompute=0, flat_allocator=allocator)
    model.init_random(42)
    model.allocate_grads()
    backend = None
    if arena is not None:
        from llmc_b200.parallel import p2p
        backend = p2p.P2PBackend(model, d, arena, bufs["params"], bufs["grads"], zero_stage=a.zero)
    opt = ShardedAdamW(model, d, a.zero, True, backend)
    B, T = 2, 64
    accum = a.slots // world
    losses = []
    for step in range(a.steps):
        if rank == a.fail_rank and step == 1:
            raise RuntimeError("injected failure on rank %d" % rank)
        for micro in range(accum):
            x, y = batch_for(step, rank * accum + micro, B, T, cfg.vocab_size)
            model.forward(x.to(d.device), y.to(d.device), accum, micro)
            model.backward(micro, micro == accum - 1)
        # norm and loss are summed over the ranks in one exchange, as in the trainer's step
        opt.grad_norm_sq(model.acts["losses"], 1.0 / float(B * T * accum))
        if step != a.skip_step:
            opt.step(1e-3, 0.1, step + 1)
        opt.backend.end_step(updated=(step != a.skip_step))
        losses.append(float(opt.scalars[1]) / world)
    if a.device == "cuda":
        from llmc_b200 import _lib
        status = _lib.read_status()
        assert status == 0, "kernel status 0x%08x on rank %d" % (status, rank)
    opt.sync_params()
    if rank == 0:
        torch.save({"params": model.params_flat.float().cpu(), "losses": losses, "backend": opt.backend.name, "zero": opt.zero_stage}, a.out)
    pdist.barrier(d)
    pdist.shutdown(d)


if __name__ == "__main__":
    main()
