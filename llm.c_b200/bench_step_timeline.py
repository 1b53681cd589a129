"""Per-phase timeline of one optimizer step on N GPUs, from CUDA events on the compute stream and on the communication
stream (max over ranks), to show where a data-parallel step spends the time that a single-GPU step does not:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29700 \\
        -m llmc_b200.bench_step_timeline --model d12 -b 64 -t 1024 --total-batch 524288

Output, rank 0, one JSON object:
  * a timeline of the LAST micro-step of the last step (ranks synchronised just before it): end of forward, end of every layer's
    backward on the compute stream, end of what the backend put on its communication stream for that layer (the flag exchange in
    the default schedule, the whole reduction with LLMC_RS_MODE=side), end of backward, of the shared group's reduction, of the
    norm / loss exchange, of the update launches, and the moment all parameters are published (max over ranks);
  * medians over the steps of the phases of a micro-step WITHOUT reductions and of the last micro-step, the exposed tail
    (end of backward to end of the norm exchange), the update launches and the whole step -- as the max over ranks and per rank.
    Ranks do not run at the same speed (power capping): a faster rank shows the difference as waiting in its last micro-step,
    so what the reductions cost is read from the SLOWEST rank's line.
The tool wraps the trainer's own objects; it changes no kernel and no schedule.
"""
import argparse
import json
import sys

import torch
import torch.distributed as dist

from .train import TrainConfig, Trainer


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="d12")
    ap.add_argument("-b", type=int, default=64)
    ap.add_argument("-t", type=int, default=1024)
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--comm", default="p2p")
    ap.add_argument("--data", default="", help="train shard pattern (default: the benchmark's synthetic shard)")
    a = ap.parse_args(argv)
    import os
    import tempfile
    pattern = a.data
    if not pattern:
        from .utils.dataloader import write_synthetic_shard
        d0 = os.path.join(tempfile.gettempdir(), "llmc_b200_timeline_data")
        os.makedirs(d0, exist_ok=True)
        path = os.path.join(d0, "synth_train_000000.bin")
        if int(os.environ.get("RANK", 0)) == 0 and not os.path.exists(path):
            write_synthetic_shard(path + ".tmp", 4 * 1024 * 1024 + 1, 50257, 1234)
            os.replace(path + ".tmp", path)
        pattern = os.path.join(d0, "synth_train_*.bin")
    cfg = TrainConfig(train_data_pattern=pattern, val_data_pattern="", load_filename=a.model, B=a.b, T=a.t, total_batch_size=a.total_batch,
                      learning_rate=6e-4, warmup_iterations=700, weight_decay=0.1, max_steps=10 ** 6, val_loss_every=0, sample_every=0,
                      recompute=0, zero_stage=1, use_master_weights=1, comm_backend=a.comm, quiet=True)
    from .parallel import dist as pdist
    dcfg = pdist.init_distributed(device_type="cuda")
    if dcfg.num_processes > 1:
        dist.barrier()
    tr = Trainer(cfg, dcfg)
    m, opt, be = tr.model, tr.opt, tr.opt.backend
    L = m.cfg.num_layers
    ev = lambda: torch.cuda.Event(enable_timing=True)
    marks = {}

    def mark(name, stream=None):
        e = ev()
        e.record(stream if stream is not None else torch.cuda.current_stream())
        marks[name] = e

    # wrap the hooks of the last micro-step
    orig_hook = m.grad_hook
    recording = {"on": False}

    def hook(layer):
        if recording["on"]:
            mark("bwd_end[%d]" % layer)
        orig_hook(layer)
        if recording["on"] and hasattr(be, "stream") and be.stream is not None:
            mark("reduce_end[%d]" % layer, be.stream)
    m.grad_hook = hook

    G = tr.grad_accum_steps
    plain_marks = None
    plain_samples, step_samples = [], []
    for step in range(a.steps):
        tl = tr.train_loader
        for micro in range(G):
            inputs, targets = tl.next_batch()
            tr._upload(inputs, targets, tl.last_index)
            last = micro == G - 1
            recording["on"] = last and step == a.steps - 1
            if recording["on"]:
                marks.clear()
                torch.cuda.synchronize()
                if dcfg.num_processes > 1:
                    dist.barrier()
                mark("start")
            plain = micro == G - 2 and step >= 2        # a micro-step without reductions, for comparison
            sampled = last and step >= 2
            if plain:
                plain_marks = [ev(), ev(), ev()]
                plain_marks[0].record()
            if sampled:
                smp = {"start": ev()}
                smp["start"].record()
            m.forward(m.inputs, m.targets, G, micro)
            if recording["on"]:
                mark("fwd_end")
            if plain:
                plain_marks[1].record()
            if sampled:
                smp["fwd"] = ev(); smp["fwd"].record()
            m.backward(micro, last_micro_step=last)
            if recording["on"]:
                mark("bwd_all_end")
            if plain:
                plain_marks[2].record()
                plain_samples.append(plain_marks)
            if sampled:
                smp["bwd"] = ev(); smp["bwd"].record()
        B_, T_ = m.act_shape
        opt.grad_norm_sq(m.acts["losses"], 1.0 / float(B_ * T_ * G))
        if recording["on"]:
            mark("norm_end")
        if step >= 2:
            smp["norm"] = ev(); smp["norm"].record()
        opt.step(6e-4, 0.1, step + 1)
        opt.backend.end_step(updated=True)
        if step >= 2:
            smp["upd"] = ev(); smp["upd"].record()
            step_samples.append(smp)
        if recording["on"]:
            mark("update_end")
            opt.sync_params()
            mark("params_complete")
        torch.cuda.synchronize()
    t0 = marks["start"]
    times = {k: t0.elapsed_time(e) for k, e in marks.items() if k != "start"}
    def median(xs):
        xs = sorted(xs)
        return xs[len(xs) // 2]
    if plain_samples:
        times["plain_fwd"] = median([p[0].elapsed_time(p[1]) for p in plain_samples])
        times["plain_bwd"] = median([p[1].elapsed_time(p[2]) for p in plain_samples])
    times["med_fwd"] = median([q["start"].elapsed_time(q["fwd"]) for q in step_samples])
    times["med_bwd"] = median([q["fwd"].elapsed_time(q["bwd"]) for q in step_samples])
    times["med_norm"] = median([q["bwd"].elapsed_time(q["norm"]) for q in step_samples])
    times["med_upd"] = median([q["norm"].elapsed_time(q["upd"]) for q in step_samples])
    # whole steps: start of the last micro-step's predecessor chain is not marked, so time consecutive "upd" events instead
    whole = [step_samples[i]["upd"].elapsed_time(step_samples[i + 1]["upd"]) for i in range(len(step_samples) - 2)]
    times["med_step"] = median(whole) if whole else 0.0
    keys = sorted(times)
    vec = torch.tensor([times[k] for k in keys], dtype=torch.float64, device=tr.device)
    per_rank = None
    if dcfg.num_processes > 1:
        gathered = [torch.zeros_like(vec) for _ in range(dcfg.num_processes)]
        dist.all_gather(gathered, vec)
        per_rank = [dict(zip(keys, [float(x) for x in g])) for g in gathered]
        dist.all_reduce(vec, op=dist.ReduceOp.MAX)
    times = dict(zip(keys, [float(x) for x in vec]))
    if dcfg.process_rank == 0:
        out = {"n_gpus": dcfg.num_processes, "model": a.model, "micro_batch": a.b, "seq_len": a.t, "grad_accum_steps": G, "comm_backend": be.name,
               "ms_since_start_of_last_micro_step (max over ranks)": {}}
        tab = out["ms_since_start_of_last_micro_step (max over ranks)"]
        tab["forward end"] = times["fwd_end"]
        for l in reversed(range(L)):
            tab["backward of layer %d end" % l] = times.get("bwd_end[%d]" % l)
            if "reduce_end[%d]" % l in times:
                tab["communication stream done for layer %d" % l] = times["reduce_end[%d]" % l]
        tab["backward end (embedding gradients)"] = times["bwd_all_end"]
        if "reduce_end[-1]" in times:
            tab["reduce of the shared group end"] = times["reduce_end[-1]"]
            tab["exposed reduce (after backward)"] = max(0.0, times["reduce_end[-1]"] - times["bwd_all_end"])
        med = out["median over steps, ms (max over ranks)"] = {}
        if "plain_bwd" in times:
            med["forward of a micro-step without reductions"] = times["plain_fwd"]
            med["backward of a micro-step without reductions"] = times["plain_bwd"]
        med["forward of the last micro-step"] = times["med_fwd"]
        med["backward of the last micro-step (layer reductions running beside it)"] = times["med_bwd"]
        med["end of backward to end of the norm / loss exchange (exposed reduction included)"] = times["med_norm"]
        med["update + all-gather launches"] = times["med_upd"]
        med["whole step (update to update, includes the host's synchronisation between steps)"] = times["med_step"]
        if per_rank is not None:
            # a rank that computes faster than its peers shows the difference as waiting in the last micro-step: read the phases
            # of the SLOWEST rank (largest plain micro-step) for what the reductions cost
            names = [("plain_fwd", "fwd plain"), ("plain_bwd", "bwd plain"), ("med_fwd", "fwd last"), ("med_bwd", "bwd last"),
                     ("med_norm", "tail+norm"), ("med_upd", "update"), ("med_step", "step")]
            out["per rank, median ms"] = {"rank %d" % r: {lab: round(pr[k], 3) for k, lab in names if k in pr} for r, pr in enumerate(per_rank)}
        tab["norm and loss all-reduce end"] = times["norm_end"]
        tab["update launches end"] = times["update_end"]
        tab["all parameters published"] = times["params_complete"]
        print(json.dumps(out, indent=1), flush=True)
    tr.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
