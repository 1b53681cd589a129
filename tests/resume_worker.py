"""Worker of the resume tests: trains through the public Trainer, optionally from a resumed state, and lets rank 0 write the
loss curve and a checksum of the final parameters.  Run directly (one process) or under torch.distributed.run."""
import argparse
import hashlib
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from llmc_b200.train import TrainConfig, Trainer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True)
    ap.add_argument("--run-name", dest="log", required=True)
    ap.add_argument("--steps", type=int, required=True)        # train until this step number
    ap.add_argument("--checkpoint-at", type=int, default=0)
    ap.add_argument("--resume", type=int, default=0)
    ap.add_argument("--backend", default="p2p")
    ap.add_argument("--zero", type=int, default=1)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    cfg = TrainConfig(train_data_pattern=os.path.join(a.dir, "train.bin"), val_data_pattern="", load_filename=os.path.join(a.dir, "init.bin"),
                      output_log_dir=os.path.join(a.dir, a.log), B=2, T=128, total_batch_size=2 * 128 * world * 2, learning_rate=1e-3,
                      weight_decay=0.1, val_loss_every=0, sample_every=0, quiet=True, tokenizer_path=os.path.join(a.dir, "none.bin"),
                      max_steps=a.steps, checkpoint_every=0, resume=a.resume, zero_stage=a.zero, comm_backend=a.backend, recompute=1)
    t = Trainer(cfg)
    losses = []
    while t.step < a.steps:
        if a.checkpoint_at and t.step == a.checkpoint_at and not t.resuming:
            t.write_checkpoint(t.step)
        losses.append(t.train_step()["loss"])
    t.opt.sync_params()
    torch.cuda.synchronize()
    digest = hashlib.sha256(t.model.params_flat.view(torch.int16).cpu().numpy().tobytes()).hexdigest()
    if t.dist.process_rank == 0:
        with open(a.out, "w") as f:
            json.dump({"losses": losses, "params": digest, "backend": t.opt.backend.name, "start": a.steps - len(losses)}, f)
    t.close()


if __name__ == "__main__":
    main()
