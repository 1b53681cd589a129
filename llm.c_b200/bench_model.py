"""Times training steps of any model descriptor on one GPU, optionally with a per-operator breakdown.

    python -m llmc_b200.bench_model --model d12 -b 64 -t 1024 --steps 5
    python -m llmc_b200.bench_model --model llama3:l=16,c=2048,h=32,kv=8,t=2048 -b 8 -t 2048 --steps 5 --ops

Every step is forward + backward + global norm + AdamW on synthetic tokens, timed with CUDA events after warm-up.  ``--ops``
adds a second pass in which every operator call is bracketed by its own pair of events (the per-kernel view that the
reference gets from profile_gpt2cu.py, without a profiler); the step time is always taken from the pass without them.
Model FLOPs utilisation is reported against ``--peak-tflops`` (default: the dense bf16 GEMM rate measured on this kind of
GPU with the vendor library, 1590 TFLOP/s).
"""
import argparse
import collections
import json
import sys

import torch


def _make_model(desc, recompute):
    from .models import gpt2, llama3
    dev = torch.device("cuda", 0)
    if desc.startswith("llama3:"):
        m = llama3.Llama(llama3.config_from_descriptor(desc), dev, torch.bfloat16, recompute=recompute)
    else:
        m = gpt2.GPT(gpt2.config_from_descriptor(desc), dev, torch.bfloat16, recompute=recompute)
    m.init_random(42)
    return m


def _instrument(records):
    """Wraps every operator so that each call leaves (tag, start event, end event) in ``records``."""
    from . import ops
    from .ops import kernels as K

    def wrap(name):
        fn = getattr(K, name)

        def w(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn(*a, **k)
            e.record()
            tag = name
            if name == "matmul_forward":
                tag += " M=%d N=%d K=%d%s" % (a[1].shape[0], a[2].shape[0], a[2].shape[1], " gelu" if k.get("pre_gelu") is not None else "")
            elif name == "matmul_dgrad":
                tag += " M=%d N=%d K=%d%s" % (a[1].shape[0], a[2].shape[1], a[2].shape[0], " dgelu" if k.get("pre_gelu") is not None else "")
            elif name == "matmul_wgrad":
                tag += " M=%d N=%d K=%d" % (a[1].shape[1], a[2].shape[1], a[1].shape[0])
            records.append((tag, s, e))
            return r
        return w

    saved = {}
    for n in ops._NAMES:
        saved[n] = (getattr(K, n), ops.__dict__[n])
        wrapped = wrap(n)
        ops.__dict__[n] = wrapped
    return saved


def _restore(saved):
    from . import ops
    for n, (_, disp) in saved.items():
        ops.__dict__[n] = disp


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="d12")
    ap.add_argument("-b", "--batch", type=int, default=64)
    ap.add_argument("-t", "--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--recompute", type=int, default=1)
    ap.add_argument("--ops", action="store_true", help="add the per-operator table")
    ap.add_argument("--peak-tflops", type=float, default=1590.0)
    a = ap.parse_args(argv)

    from .parallel.dist import DistConfig
    from .parallel.zero import ShardedAdamW
    m = _make_model(a.model, a.recompute)
    dev = m.device
    opt = ShardedAdamW(m, DistConfig(0, 1, 0, dev), 0, True)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, m.cfg.vocab_size, (a.batch, a.seq + 1), generator=g, dtype=torch.int32)
    x, y = tok[:, :-1].contiguous().to(dev), tok[:, 1:].contiguous().to(dev)

    def step(i):
        m.forward(x, y)
        m.backward()
        opt.grad_norm_sq()
        opt.step(3e-4, 0.1, i + 1)

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        step(a.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    tokens = a.batch * a.seq
    tflops = m.flops_per_token(a.seq) * tokens / (ms * 1e-3) / 1e12
    out = {"model": a.model, "parameters": m.num_parameters, "batch": a.batch, "seq_len": a.seq, "recompute": a.recompute,
           "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3), "model_tflops": tflops, "mfu_of_peak": tflops / a.peak_tflops,
           "loss": float(m.loss()), "memory_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    print(json.dumps(out))

    if a.ops:
        records = []
        saved = _instrument(records)
        try:
            for i in range(2):
                records.clear()
                m.forward(x, y)
                m.backward()
                torch.cuda.synchronize()
        finally:
            _restore(saved)
        agg = collections.OrderedDict()
        for tag, s, e in records:
            cell = agg.setdefault(tag, [0, 0.0])
            cell[0] += 1
            cell[1] += s.elapsed_time(e)
        total = sum(v[1] for v in agg.values())
        print("forward + backward, sum of operator times %.2f ms" % total)
        for tag, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            print("%-52s n=%4d total %9.3f ms  avg %8.3f ms  %5.1f%%" % (tag, n, t, t / n, 100 * t / total))
    return 0


if __name__ == "__main__":
    sys.exit(main())
