"""Post-processes an ``ncu`` capture of a training step into per-kernel and per-phase tables
(reference: profile_gpt2cu.py, which drives ncu on profile_gpt2.cu).

    # on the GPU box, one process, small model, the plain run first:
    python -m llmc_b200.profile_step run                      # one step of a 1-layer GPT-2 124M-width model, B=24 T=1024
    ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv python -m llmc_b200.profile_step run
    # anywhere:
    python -m llmc_b200.profile_step report launches.csv
    # with more columns (several passes per launch: keep the model at one layer):
    ncu --metrics gpu__time_duration.sum,dram__bytes_read.sum,dram__bytes_write.sum,sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active,smsp__inst_executed.sum \
        --clock-control none --csv --log-file launches.csv python -m llmc_b200.profile_step run

``report`` takes the last optimizer step of the capture, classifies its launches into encoder / forward / classifier /
backward / optimizer phases, scales the per-layer phases to the 12 layers of the 124M model and prints per-kernel and
per-phase time, DRAM traffic, tensor-pipe activity and an efficiency score (reference: profile_gpt2cu.py:36-228).
It reads only the CSV; nothing is disassembled.
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


# metrics the report understands (ask ncu for any subset; time alone is a one-pass capture)
METRICS = ["gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "lts__t_sectors_srcunit_tex_op_read.sum",
           "lts__t_sectors_srcunit_tex_op_write.sum", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
           "smsp__inst_executed.sum"]


def _num(x):
    try:
        return float(str(x).replace(",", ""))
    except ValueError:
        return 0.0


def read_launches(path):
    """Launches in order as dicts {name, metric: value}.  Accepts both layouts ncu writes: one row per (launch, metric)
    (``--csv --log-file`` of a capture with ``--metrics``) and one row per launch with a column per metric (``--page raw --csv``)."""
    with open(path) as f:
        lines = [l for l in f if not l.startswith("==")]
    rows = list(csv.reader(lines))
    if not rows:
        return []
    head = rows[0]
    launches = []
    if "Metric Name" in head:
        ix = {h: i for i, h in enumerate(head)}
        by_id = collections.OrderedDict()
        for r in rows[1:]:
            if len(r) != len(head):
                continue
            d = by_id.setdefault(r[ix["ID"]], {"name": r[ix["Kernel Name"]]})
            v = _num(r[ix["Metric Value"]])
            unit = r[ix.get("Metric Unit", 0)] if "Metric Unit" in ix else ""
            name = r[ix["Metric Name"]]
            if name == "gpu__time_duration.sum":
                v *= {"ns": 1.0, "us": 1e3, "usecond": 1e3, "ms": 1e6, "msecond": 1e6, "second": 1e9, "s": 1e9}.get(unit, 1.0)
            if name.startswith("dram__bytes"):
                v *= {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(unit, 1.0)
            d[name] = v
        launches = list(by_id.values())
    else:
        units = rows[1] if len(rows) > 1 else []
        ix = {h: i for i, h in enumerate(head)}
        for r in rows[2:]:
            if len(r) != len(head):
                continue
            d = {"name": r[ix.get("Kernel Name", 0)]}
            for m in METRICS:
                if m in ix:
                    v = _num(r[ix[m]])
                    unit = units[ix[m]] if units else ""
                    if m == "gpu__time_duration.sum":
                        v *= {"ns": 1.0, "us": 1e3, "usecond": 1e3, "ms": 1e6, "msecond": 1e6}.get(unit, 1.0)
                    if m.startswith("dram__bytes"):
                        v *= {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(unit, 1.0)
                    d[m] = v
            launches.append(d)
    return launches


def short_name(name):
    return name.split("(")[0].replace("void ", "").replace("<unnamed>::", "").strip()


def classify(launches):
    """Phase of every launch of ONE training step of run_step(): enc (embedding lookup), fwd (the layers), cls (LM head and loss),
    bwd (everything up to the embedding gradients), opt (norm and AdamW).  Decided by kernel name and position, as the
    reference's tool does by launch index (profile_gpt2cu.py:96-118)."""
    phases = []
    phase = "enc"
    seen_cls = False
    for l in launches:
        n = short_name(l["name"])
        if phase == "enc" and not n.startswith("encoder_fwd"):
            phase = "fwd"
        if "classifier" in n:
            phase, seen_cls = "cls", True
        elif phase == "cls" and seen_cls and not n.startswith("gemm"):
            phase = "bwd"
        if "norm_sq" in n or n.startswith("adamw") or n.startswith("final_sum"):
            phase = "opt"
        phases.append(phase)
    # the LM-head GEMM runs right before the classifier: it belongs to cls
    for k in range(len(launches) - 1):
        if phases[k] == "fwd" and phases[k + 1] == "cls":
            phases[k] = "cls"
    # the GEMMs right after the classifier are the LM head's backward (dgrad, wgrad): they stay in cls (one per model, not per
    # layer); everything after the first other kernel is bwd
    k = 0
    while k < len(phases) and "classifier" not in short_name(launches[k]["name"]):
        k += 1
    m = k + 1
    while m < len(phases) and short_name(launches[m]["name"]).startswith("gemm"):
        phases[m] = "cls"
        m += 1
    for q in range(m, len(phases)):
        if phases[q] == "cls":
            phases[q] = "bwd"
    return phases


def report(path, out=sys.stdout, layers_profiled=1, layers_model=12, hbm_gbs=6542.4, step=-1):
    """Per-kernel and per-phase tables of the LAST optimizer step in the capture (earlier steps are warm-up).  The per-layer
    phases (fwd, bwd) are scaled from the profiled layer count to ``layers_model``, like the reference's summary; DRAM traffic,
    tensor-pipe activity and instruction counts are shown when the capture has them.  ``efficiency`` is the time-weighted
    mean of max(DRAM bandwidth fraction, tensor-pipe fraction) per kernel: how close the step runs to one of its two roofs."""
    launches = read_launches(path)
    launches = [l for l in launches if "gpu__time_duration.sum" in l]
    if not launches:
        print("no kernel rows found in %s" % path, file=out)
        return {}
    # split into steps at every embedding lookup
    starts = [k for k, l in enumerate(launches) if short_name(l["name"]).startswith("encoder_fwd")]
    if starts:
        s0 = starts[step]
        later = [x for x in starts if x > s0]
        launches = launches[s0:(later[0] if later else len(launches))]
    phases = classify(launches)
    have_dram = any("dram__bytes_read.sum" in l for l in launches)
    have_tc = any(METRICS[5] in l for l in launches)
    per = collections.OrderedDict()
    for l, ph in zip(launches, phases):
        a = per.setdefault((ph, short_name(l["name"])), dict(n=0, t=0.0, rd=0.0, wr=0.0, tc=0.0, inst=0.0))
        a["n"] += 1
        a["t"] += l["gpu__time_duration.sum"]
        a["rd"] += l.get("dram__bytes_read.sum", 0.0)
        a["wr"] += l.get("dram__bytes_write.sum", 0.0)
        a["tc"] += l.get(METRICS[5], 0.0) * l["gpu__time_duration.sum"]
        a["inst"] += l.get("smsp__inst_executed.sum", 0.0)
    scale = {"fwd": layers_model / layers_profiled, "bwd": layers_model / layers_profiled}
    print("%-5s %-44s %5s %10s %9s %9s %8s %9s" % ("phase", "kernel", "count", "time (us)", "DRAM rd MB", "DRAM wr MB", "tensor %", "DRAM GB/s"), file=out)
    tot = collections.OrderedDict((ph, dict(t=0.0, rd=0.0, wr=0.0, eff=0.0)) for ph in ("enc", "fwd", "cls", "bwd", "opt"))
    for (ph, k), a in per.items():
        bw = (a["rd"] + a["wr"]) / a["t"] if a["t"] > 0 else 0.0          # bytes per ns = GB/s
        tcp = a["tc"] / a["t"] if a["t"] > 0 else 0.0
        print("%-5s %-44s %5d %10.1f %9s %9s %8s %9s" % (ph, k[:44], a["n"], a["t"] / 1e3,
              ("%.1f" % (a["rd"] / 1e6)) if have_dram else "-", ("%.1f" % (a["wr"] / 1e6)) if have_dram else "-",
              ("%.1f" % tcp) if have_tc else "-", ("%.0f" % bw) if have_dram else "-"), file=out)
        f = scale.get(ph, 1.0)
        tot[ph]["t"] += a["t"] * f
        tot[ph]["rd"] += a["rd"] * f
        tot[ph]["wr"] += a["wr"] * f
        tot[ph]["eff"] += a["t"] * f * max(min(bw / hbm_gbs, 1.0), tcp / 100.0)
    total = sum(v["t"] for v in tot.values())
    print("\nsummary for %d layers (fwd and bwd scaled from %d profiled):" % (layers_model, layers_profiled), file=out)
    print("%-5s %12s %7s %12s %12s" % ("phase", "time (ms)", "share", "DRAM rd GB", "DRAM wr GB"), file=out)
    for ph, v in tot.items():
        print("%-5s %12.3f %6.1f%% %12s %12s" % (ph, v["t"] / 1e6, 100 * v["t"] / total if total else 0.0,
              ("%.2f" % (v["rd"] / 1e9)) if have_dram else "-", ("%.2f" % (v["wr"] / 1e9)) if have_dram else "-"), file=out)
    print("total %.3f ms" % (total / 1e6), file=out)
    if have_dram or have_tc:
        print("efficiency %.1f%% (time-weighted max of DRAM-bandwidth and tensor-pipe fraction per kernel; HBM peak %.0f GB/s)"
              % (100 * sum(v["eff"] for v in tot.values()) / total, hbm_gbs), file=out)
    return dict(kernels=per, phases=tot, total_ns=total)


if __name__ == "__main__":
    if len(sys.argv) >= 2 and sys.argv[1] == "run":
        run_step()
    elif len(sys.argv) >= 3 and sys.argv[1] == "report":
        report(sys.argv[2])
    else:
        print(__doc__)
