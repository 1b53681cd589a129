"""Post-processes an ``ncu`` capture of a training step into per-kernel and per-phase tables
(reference: profile_gpt2cu.py, which drives ncu on profile_gpt2.cu).

    # on the GPU box, one process, small model, the plain run first:
    python -m llmc_b200.profile_step run                      # one step of a 1-layer GPT-2 124M-width model, B=24 T=1024
    ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv python -m llmc_b200.profile_step run
    # anywhere:
    python -m llmc_b200.profile_step report launches.csv

``report`` sums device time per kernel name and classifies kernels into encoder / forward / classifier / backward /
optimizer phases by launch order, like the reference's tool.  It reads only the CSV; nothing is disassembled.
"""
import collections
import csv
import sys


def run_step(layers=1, B=24, T=1024):
    import torch
    from .models import gpt2
    from .parallel.dist import DistConfig
    from .parallel.zero import ShardedAdamW
    cfg = gpt2.GPTConfig(1024, 50257, 50304, layers, 12, 768)
    dev = torch.device("cuda", 0)
    model = gpt2.GPT(cfg, dev, torch.bfloat16, recompute=1)
    model.init_random(42)
    opt = ShardedAdamW(model, DistConfig(0, 1, 0, dev), 0, True)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g, dtype=torch.int32)
    x, y = tok[:, :-1].contiguous().to(dev), tok[:, 1:].contiguous().to(dev)
    for step in range(2):
        torch.cuda.nvtx.range_push("step %d" % step)
        model.forward(x, y)
        model.backward()
        opt.grad_norm_sq()
        opt.step(3e-4, 0.0, step + 1)
        torch.cuda.nvtx.range_pop()
    torch.cuda.synchronize()
    print("loss %.4f" % float(model.loss()))


def report(path, out=sys.stdout):
    rows = []
    with open(path) as f:
        lines = [l for l in f if not l.startswith("==")]
    rd = csv.DictReader(lines)
    for r in rd:
        name = r.get("Kernel Name") or r.get("Name") or ""
        val = r.get("Metric Value") or r.get("gpu__time_duration.sum") or "0"
        try:
            rows.append((name, float(val.replace(",", ""))))
        except ValueError:
            continue
    if not rows:
        print("no kernel rows found in %s" % path, file=out)
        return {}
    per = collections.OrderedDict()
    for name, t in rows:
        short = name.split("(")[0].replace("void ", "").replace("<unnamed>::", "")
        a = per.setdefault(short, [0, 0.0])
        a[0] += 1
        a[1] += t
    total = sum(v[1] for v in per.values())
    print("%-60s %6s %12s %7s" % ("kernel", "count", "time (us)", "share"), file=out)
    for k, (n, t) in sorted(per.items(), key=lambda kv: -kv[1][1]):
        print("%-60s %6d %12.1f %6.1f%%" % (k[:60], n, t / 1e3, 100 * t / total), file=out)
    print("total device time %.3f ms over %d launches" % (total / 1e6, len(rows)), file=out)
    return per


if __name__ == "__main__":
    if len(sys.argv) >= 2 and sys.argv[1] == "run":
        run_step()
    elif len(sys.argv) >= 3 and sys.argv[1] == "report":
        report(sys.argv[2])
    else:
        print(__doc__)
