"""Times generation with the key / value cache on one GPU.

    python -m llmc_b200.bench_generate --model llama3:l=16,c=2048,h=32,kv=8,t=2048 --batch 4 --prompt 128 --gen 64

Prefill (all prompt tokens at once) and decoding (one token per row and step) are timed separately with CUDA events after a
warm-up pass.  A decoding step reads every weight once, so its floor is (parameter bytes + cache bytes read) / memory
bandwidth; the achieved fraction is printed against ``--peak-gbs`` (default: the copy bandwidth measured on this kind of GPU).
Greedy sampling, random weights, synthetic prompts.
"""
import argparse
import json
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="llama3:l=16,c=2048,h=32,kv=8,t=2048")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--gen", type=int, default=64)
    ap.add_argument("--graph", type=int, default=1, help="replay the one-token step from a CUDA graph (0: launch every kernel each step)")
    ap.add_argument("--peak-gbs", type=float, default=6542.0)
    a = ap.parse_args(argv)

    from .models import generate as G
    from .models import llama3
    dev = torch.device("cuda", 0)
    m = llama3.Llama(llama3.config_from_descriptor(a.model), dev, torch.bfloat16, recompute=1)
    m.init_random(42)
    cfg = m.cfg
    total = a.prompt + a.gen
    dec = G.CachedDecoder(m, a.batch, total)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=g, dtype=torch.int32).to(dev)

    def run(timed):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        logits = dec.forward(prompt, 0)
        ev[1].record()
        if a.graph:
            gs.pos.fill_(a.prompt)
        for t in range(a.prompt, total):
            nxt = torch.argmax(logits, dim=-1).to(torch.int32).view(a.batch, 1)
            logits = gs.step(nxt) if a.graph else dec.forward(nxt, t)
        ev[2].record()
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2]) / a.gen

    gs = G.GraphStep(dec, a.batch, a.prompt) if a.graph else None
    run(False)
    prefill_ms, step_ms = run(True)
    weight_bytes = 2 * (m.num_parameters - cfg.padded_vocab_size * cfg.channels)       # the embedding table is gathered, not streamed
    cache_bytes = dec.cache_bytes() * (a.prompt + a.gen / 2) / total
    out = {"model": a.model, "parameters": m.num_parameters, "batch": a.batch, "prompt": a.prompt, "gen": a.gen, "cuda_graph": bool(a.graph),
           "prefill_ms": prefill_ms, "prefill_tokens_per_s": a.batch * a.prompt / (prefill_ms * 1e-3),
           "decode_ms_per_step": step_ms, "decode_tokens_per_s": a.batch / (step_ms * 1e-3),
           "decode_gbs": (weight_bytes + cache_bytes) / (step_ms * 1e-3) / 1e9,
           "decode_fraction_of_peak_bandwidth": (weight_bytes + cache_bytes) / (step_ms * 1e-3) / 1e9 / a.peak_gbs,
           "cache_mib": dec.cache_bytes() / 2 ** 20}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
