"""LLaMA-3 training / fine-tuning on B200 with the long options of the reference's PyTorch script (train_llama3.py:940-975
of the reference), driven by this framework's engine instead of torch.nn / autograd:

    python train_llama3.py --model llama3:8B --input_bin 'data/train_*.bin' --input_val_bin 'data/val_*.bin' \
        --batch_size 1 --sequence_length 8192 --total_batch_size 65536 --zero_stage 1 --num_iterations 100
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 train_llama3.py --model llama3:8B --zero_stage 1 ...

``--model`` takes a model file written by ``utils.checkpoint.write_model`` or by the reference's ``write_model`` (magic
20240803), or a descriptor (``llama3:8B``, ``llama3:70B``, ``llama3:405B``, ``llama3:l=..,c=..,h=..,kv=..``) for random
initialisation; the Hugging Face id ``meta-llama/Meta-Llama-3.1-8B`` is accepted as an alias of ``llama3:8B`` (pretrained weights
need a download, so they enter through a model file).  Token shards are the 32-bit files of the reference
(magic 20240801).  ``--write_tensors 1`` writes the model file and the debug-state file (inputs, targets, logits, loss and
all gradients of the first batch, fp32) that the reference script writes for cross-checking other implementations.
``--inference_only 1`` reports the validation loss and generates from ``--prompt_tokens`` (batched prompts as token ids, key /
value cache, nucleus sampling at ``--temperature`` / ``--top_p``; ``--use_kv 0`` recomputes the prefix instead).
"""
import argparse
import os
import sys

import numpy as np
import torch

from llmc_b200.train import TrainConfig, Trainer
from llmc_b200.utils import checkpoint

ALIASES = {"meta-llama/Meta-Llama-3.1-8B": "llama3:8B", "meta-llama/Meta-Llama-3.1-70B": "llama3:70B",
           "meta-llama/Meta-Llama-3.1-405B": "llama3:405B"}


def build_parser():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--input_bin", type=str, default="dev/data/tinyshakespeare/tiny_shakespeare_val.bin")
    p.add_argument("--input_val_bin", type=str, default="")
    p.add_argument("--output_dir", type=str, default="")
    p.add_argument("--model", type=str, default="meta-llama/Meta-Llama-3.1-8B")
    p.add_argument("--tokenizer_path", type=str, default="llama3_tokenizer.bin")
    p.add_argument("--batch_size", type=int, default=4)
    p.add_argument("--sequence_length", type=int, default=64)
    p.add_argument("--total_batch_size", type=int, default=256)
    p.add_argument("--num_iterations", type=int, default=10)
    p.add_argument("--inference_only", type=int, default=0)
    p.add_argument("--learning_rate", type=float, default=1e-5)
    p.add_argument("--warmup_iters", type=int, default=0)
    p.add_argument("--learning_rate_decay_frac", type=float, default=1.0)
    p.add_argument("--weight_decay", type=float, default=0.0)
    p.add_argument("--grad_clip", type=float, default=1.0)
    p.add_argument("--val_loss_every", type=int, default=0)
    p.add_argument("--val_max_steps", type=int, default=20)
    p.add_argument("--sample_every", type=int, default=0)
    p.add_argument("--overfit_single_batch", type=int, default=1)
    p.add_argument("--tensorcores", type=int, default=1, help="accepted for compatibility; the bf16 path always runs on tensor cores")
    p.add_argument("--device", type=str, default="")
    p.add_argument("--compile", type=int, default=0, help="accepted for compatibility; there is no tracing compiler in this framework")
    p.add_argument("--dtype", type=str, default="bfloat16", help="float32 (CPU path) | bfloat16")
    p.add_argument("--zero_stage", type=int, default=0)
    p.add_argument("--recompute", type=int, default=1)
    p.add_argument("--checkpoint_every", type=int, default=0)
    p.add_argument("--resume", type=int, default=0)
    p.add_argument("--write_tensors", type=int, default=0)
    p.add_argument("--prompt_tokens", type=str, default="", help="prompts for --inference_only as token ids, e.g. '128000,9906;128000,791' "
                   "(the tokenizer file of this framework only decodes)")
    p.add_argument("--max_gen_len", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.6)
    p.add_argument("--top_p", type=float, default=0.9)
    p.add_argument("--use_kv", type=int, default=1, help="0: recompute the prefix for every token instead of caching keys and values")
    p.add_argument("--watchdog_s", type=float, default=0.0, help="end the process if no optimizer step completes within this many seconds")
    return p


def train_config(args):
    model = ALIASES.get(args.model, args.model)
    if not (model.endswith(".bin") or model.startswith("llama3:")):
        raise SystemExit("--model must be a model file or a llama3: descriptor, got %r" % args.model)
    dtype = {"float32": "fp32", "bfloat16": "bf16"}.get(args.dtype)
    if dtype is None:
        raise SystemExit("--dtype must be float32 or bfloat16 (float16 has no kernels here)")
    return TrainConfig(
        train_data_pattern=args.input_bin, val_data_pattern=args.input_val_bin, load_filename=model, output_log_dir=args.output_dir,
        B=args.batch_size, T=args.sequence_length, total_batch_size=args.total_batch_size, max_steps=args.num_iterations,
        learning_rate=args.learning_rate, warmup_iterations=args.warmup_iters, final_learning_rate_frac=args.learning_rate_decay_frac,
        weight_decay=args.weight_decay, grad_clip=args.grad_clip, val_loss_every=args.val_loss_every, val_max_steps=args.val_max_steps,
        sample_every=args.sample_every, overfit_single_batch=args.overfit_single_batch, device=args.device, dtype=dtype,
        zero_stage=args.zero_stage, recompute=args.recompute, checkpoint_every=args.checkpoint_every, resume=args.resume,
        tokenizer_path=args.tokenizer_path, beta2=0.95, watchdog_s=args.watchdog_s)


def write_debug_state(trainer, model_path, state_path):
    """Model file plus the reference's debug-state layout (train_llama3.py:907-930 of the reference): header {20240803, B, T},
    x, y (int32), logits (fp32, unpadded vocabulary), loss, gradients in file order (fp32)."""
    m = trainer.model
    checkpoint.write_model(model_path, m)
    inputs, targets = trainer.train_loader.next_batch()
    trainer.train_loader.reset()
    x, y = inputs.to(m.device), targets.to(m.device)
    m.forward(x, y, write_dlogits=False)
    B, T = x.shape
    V = m.cfg.vocab_size
    logits = m.logits()[..., :V].float().cpu()
    m.forward(x, y)
    m.backward()
    loss = float(m.loss())
    header = np.zeros(256, dtype=np.int32)
    header[:3] = [20240803, B, T]
    grads_model = type("G", (), {"params": m.grads, "cfg": m.cfg})
    with open(state_path, "wb") as f:
        f.write(header.tobytes())
        f.write(inputs.numpy().astype(np.int32).tobytes())
        f.write(targets.numpy().astype(np.int32).tobytes())
        f.write(logits.numpy().tobytes())
        f.write(np.float32(loss).tobytes())
        Vp = m.cfg.padded_vocab_size
        for t in checkpoint._llama_file_tensors(grads_model):
            if t.dim() == 2 and t.shape[0] == Vp and Vp != V:
                t = t[:V]
            f.write(t.float().cpu().numpy().tobytes())
    return loss


def generate_from_args(model, args):
    """Batched generation as in the reference's sampling block (train_llama3.py:1150-1178), prompts given as token ids."""
    from llmc_b200.models.generate import generate
    V = model.cfg.vocab_size
    if args.prompt_tokens:
        prompts = [[int(t) for t in row.split(",") if t.strip()] for row in args.prompt_tokens.split(";") if row.strip()]
    else:
        prompts = [[min(128000, V - 1)]]
    stops = [t for t in (128001, 128009) if t < V]
    gen = torch.Generator().manual_seed(1337)
    return generate(model, prompts, args.max_gen_len, temperature=args.temperature, top_p=args.top_p, stop_tokens=stops,
                    generator=gen, use_kv=bool(args.use_kv))


def main(argv=None):
    args = build_parser().parse_args(argv)
    cfg = train_config(args)
    trainer = Trainer(cfg)
    try:
        if args.write_tensors and trainer.dist.process_rank == 0:
            tag = "bf16" if trainer.model.dtype == torch.bfloat16 else "fp32"
            out = args.output_dir or "."
            os.makedirs(out, exist_ok=True)
            loss = write_debug_state(trainer, os.path.join(out, "llama3_%s.bin" % tag), os.path.join(out, "llama3_debug_state.bin"))
            trainer.print0("wrote model and debug state (loss %.6f) to %s" % (loss, out))
        if args.inference_only:
            if trainer.val_loader is not None:
                trainer.print0("val loss %f" % trainer.validate())
            if trainer.dist.process_rank == 0:
                for toks in generate_from_args(trainer.model, args):
                    trainer.print0("generated token ids: " + " ".join(str(int(t)) for t in toks))
        else:
            trainer.run()
    finally:
        trainer.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
