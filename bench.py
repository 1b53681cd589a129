"""Headline benchmark: GPT-2 124M training throughput (tokens/s) on 1/2/4/8 B200.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...        # the unmodified reference trainer built under baseline/_ref

Configuration (the reference's scripts/run_gpt2_124M.sh): GPT-2 124M (d12), bf16, micro-batch 64 x 1024 per GPU, 524288
tokens per optimizer step through gradient accumulation, ZeRO-1, AdamW lr 6e-4 with 700 warm-up steps, weight decay
0.1, gradient clipping 1.0, fp32 master weights with stochastic rounding; random-init weights and seeded uniform-random
uint16 tokens (no datasets are available offline).

Two timed regions, both K full optimizer steps, both bracketed by barrier + synchronize, max over ranks:
  value   device time (CUDA events) of K steps driven from token batches that already sit in device memory;
  e2e     wall time of K ``Trainer.train_step()`` calls: C++ loader -> pinned host buffers -> H2D copy each micro-step,
          loss and gradient norm read back to the host each step.
One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "gpt2_124M_train_tokens_per_sec"
PUBLISHED_BASELINE = 1.75e6     # tok/s, 8 x A100 80GB, reference scripts/run_gpt2_124M.sh:4-6 (derived from ~300 ms/iter)
MODELS = {"d12": "gpt2_124M", "d24": "gpt2_350M", "d36": "gpt2_774M", "d48": "gpt2_1558M"}


def metric_name(model):
    """The headline metric is named for the model it was measured on (the published baseline number exists for d12 only)."""
    return METRIC if model == "d12" else "%s_train_tokens_per_sec" % MODELS.get(model, model)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="d12")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--recompute", type=int, default=0)
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--zero", type=int, default=1)
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi (read only) while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []
        self.nvml_samples, self.nvml_stop, self.thread = None, None, None

    def _nvml_loop(self, pynvml, handle):
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.nvml_stop.is_set():
            try:
                mask = reasons_fn(handle)
                self.nvml_samples.append((float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                          float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                          pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0, [n for bit, n in names.items() if mask & bit]))
            except Exception:
                pass
            time.sleep(0.025)

    def start(self):
        # NVML in-process (read-only queries every 25 ms: short multi-GPU steps still get a few samples); nvidia-smi otherwise
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml_samples, self.nvml_stop = [], threading.Event()
            self.thread = threading.Thread(target=self._nvml_loop, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml_samples = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml_samples is not None:
            self.nvml_stop.set()
            self.thread.join(timeout=2)
            smp = self.nvml_samples
            if not smp:
                return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
            return {"sm_mhz": statistics.median(x[0] for x in smp), "sm_max_mhz": max(x[1] for x in smp),
                    "power_w_max": max(x[2] for x in smp), "samples": len(smp), "reasons": sorted({r for x in smp for r in x[3]})}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, maxc, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0])); maxc.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxc), "power_w_max": max(power), "samples": len(clocks),
                "reasons": sorted(reasons)}


MAX_RANKS = 8     # shards are sized for the largest run of one node, whatever the world size of this run


def shard_sizes(a):
    """Token counts of the synthetic shards.  They depend on the batch geometry only, never on the world size, and are part
    of the file names: a file left behind by a run with another geometry or rank count can neither be reused by mistake
    nor be too small for a loader that wants world * B * T + 1 tokens (the reference's dataloader.h:186 asserts that)."""
    ntok_train = max(2 * a.total_batch + 1, MAX_RANKS * a.batch * a.seq * 2 + 1, 4 * 1024 * 1024)
    ntok_val = MAX_RANKS * a.batch * a.seq * 2 + 1
    return ntok_train, ntok_val


def write_shards(a, seed=1234):
    """Writes (once) the train and validation shard of this geometry; returns (directory, train pattern, val pattern)."""
    from llmc_b200.utils.dataloader import write_synthetic_shard
    ntok_train, ntok_val = shard_sizes(a)
    directory = os.path.join(tempfile.gettempdir(), "llmc_b200_bench_data", "tr%d_va%d" % (ntok_train, ntok_val))
    os.makedirs(directory, exist_ok=True)
    for name, ntok, sd in (("synth_train_000000.bin", ntok_train, seed), ("synth_val_000000.bin", ntok_val, seed + 1)):
        path = os.path.join(directory, name)
        want = 256 * 4 + 2 * ntok
        if not os.path.exists(path) or os.path.getsize(path) != want:
            tmp = "%s.tmp%d" % (path, os.getpid())
            write_synthetic_shard(tmp, ntok, 50257, sd)
            os.replace(tmp, path)
    return directory


def shard_patterns(a):
    ntok_train, ntok_val = shard_sizes(a)
    directory = os.path.join(tempfile.gettempdir(), "llmc_b200_bench_data", "tr%d_va%d" % (ntok_train, ntok_val))
    return os.path.join(directory, "synth_train_*.bin"), os.path.join(directory, "synth_val_*.bin")


def config_record(a, world, zero_stage):
    """The workload description; both arms print exactly these keys so that their records can be compared field by field."""
    return {"model": MODELS.get(a.model, a.model), "global_batch": a.total_batch, "micro_batch_per_gpu": a.batch, "seq_len": a.seq,
            "grad_accum_steps": a.total_batch // (a.batch * a.seq * world),
            "parallelism": ("dp%d-zero%d" % (world, zero_stage)) if world > 1 else "single", "recompute": a.recompute,
            "optimizer": "AdamW fp32 master + stochastic rounding",
            "l2": "no flush: every kernel's working set (activations 20+ GB per micro-step) exceeds the 126 MB L2"}


def mfu_measured(model_flops_per_gpu):
    """Model FLOP/s per GPU as a fraction of the sustained bf16 matmul peak measured on this machine class (MEASURED_PEAKS.json at
    the repository root, written by the benchmark driver); None if that file is absent."""
    from llmc_b200.utils import mfu
    peak = mfu.measured_peak_tflops()
    return model_flops_per_gpu / (peak * 1e12) if peak > 0 else None


def env_rank():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


# ----------------------------------------------------------------------------------------------- our arm
def run_ours(a):
    import torch
    import torch.distributed as dist
    from llmc_b200.ops import kernels
    from llmc_b200.train import TrainConfig, Trainer

    rank, world, local = env_rank()
    if world != a.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE is %d: launch with torch.distributed.run" % (a.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    if rank == 0:
        write_shards(a)
    cfg = TrainConfig(train_data_pattern=shard_patterns(a)[0], val_data_pattern="", load_filename=a.model,
                      B=a.batch, T=a.seq, total_batch_size=a.total_batch, learning_rate=6e-4, warmup_iterations=700,
                      final_learning_rate_frac=0.0, weight_decay=0.1, max_steps=10 ** 6, val_loss_every=0, sample_every=0,
                      recompute=a.recompute, zero_stage=a.zero, use_master_weights=1, comm_backend=a.comm, quiet=True)
    # all ranks need the shard before building the loader
    from llmc_b200.parallel import dist as pdist
    dcfg = pdist.init_distributed(device_type="cuda")
    if world > 1:
        dist.barrier()
    trainer = Trainer(cfg, dcfg)
    model, opt = trainer.model, trainer.opt
    dev = trainer.device
    G = trainer.grad_accum_steps

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- region A: device-timed, batches resident on the device
    gen = torch.Generator(device="cpu").manual_seed(4321 + rank)
    resident = [torch.randint(0, 50257, (a.batch, a.seq + 1), generator=gen, dtype=torch.int32).to(dev) for _ in range(G)]

    def device_step(step):
        for micro in range(G):
            model.inputs.copy_(resident[micro][:, :-1])
            model.targets.copy_(resident[micro][:, 1:])
            model.forward(model.inputs, model.targets, G, micro)
            model.backward(micro, last_micro_step=(micro == G - 1))
        opt.grad_norm_sq(model.acts["losses"], 1.0 / float(a.batch * a.seq * G))      # norm and loss, summed over the ranks
        opt.step(trainer.scheduler.get_learning_rate(step), cfg.weight_decay, step + 1)
        opt.backend.end_step(updated=True)

    for s in range(a.warmup):
        device_step(s)
    sync_all()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = kernels.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for s in range(a.steps):
        device_step(a.warmup + s)
    ev1.record()
    sync_all()
    dev_ms = ev0.elapsed_time(ev1)
    launches = kernels.launch_count() - launches0
    clocks = sampler.stop()

    # ---- region B: end to end through the public API
    trainer.step = a.warmup + a.steps
    for _ in range(max(1, min(a.warmup, 2))):
        trainer.train_step()
    sync_all()
    t0 = time.perf_counter()
    last = None
    for _ in range(a.steps):
        last = trainer.train_step()
    sync_all()
    e2e_s = time.perf_counter() - t0

    times = torch.tensor([dev_ms, e2e_s * 1000.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    from llmc_b200 import _lib
    status = _lib.read_status()
    tokens = a.total_batch * a.steps
    value = tokens / (dev_ms / 1000.0)
    e2e_value = tokens / (e2e_ms / 1000.0)
    flops_tok = model.flops_per_token(a.seq)
    if rank == 0:
        out = {
            "metric": metric_name(a.model), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": dev_ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": (value / PUBLISHED_BASELINE if a.model == "d12" else None),
            "dtype": "bf16", "data": "synthetic (seeded uniform-random uint16 tokens, random-init weights)",
            "config": config_record(a, world, opt.zero_stage),
            "comm_backend": opt.backend.name,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / a.steps,
                    "h2d_bytes_per_step": G * 2 * a.batch * a.seq * 4, "d2h_bytes_per_step": 8, "loss": last["loss"] if last else None},
            "gpu_launches": launches,
            "mfu_vs_2250_tflops": value / world * flops_tok / 2.25e15,
            "mfu_vs_measured_sustained_peak": mfu_measured(value / world * flops_tok),
            "kernel_status": status,
            "impl": "ours",
        }
        print(json.dumps(out), flush=True)
    trainer.close()


# ----------------------------------------------------------------------------------------------- reference arm
def run_reference(a):
    rank, world, local = env_rank()
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    exe = os.path.join(ref_dir, "train_gpt2cu")

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    if not os.path.exists(exe):
        return unavailable("baseline/_ref/train_gpt2cu is not built (see baseline/README.md)")
    sync_dir = os.path.join(tempfile.gettempdir(), "llmc_b200_ref_sync_%s" % os.environ.get("MASTER_PORT", "0"))
    if rank == 0:
        write_shards(a)
        os.makedirs(sync_dir, exist_ok=True)
        stale = os.path.join(sync_dir, "ncclUniqueId.sync")
        if os.path.exists(stale):
            os.remove(stale)
        open(os.path.join(sync_dir, "ready"), "w").close()
    else:
        for _ in range(600):
            if os.path.exists(os.path.join(sync_dir, "ready")):
                break
            time.sleep(0.1)
    total_steps = a.warmup + a.steps
    train_pattern, val_pattern = shard_patterns(a)
    cmd = [exe, "-i", train_pattern, "-j", val_pattern, "-e", a.model,
           "-b", str(a.batch), "-t", str(a.seq), "-d", str(a.total_batch), "-z", str(a.zero), "-c", "0.1", "-l", "6e-4", "-u", "700", "-q", "0.0",
           "-r", str(a.recompute), "-x", str(total_steps), "-v", "1000000", "-m", "1", "-s", "1000000", "-g", "2", "-h", "0", "-n", "0"]
    # the reference's default rendezvous is MPI, which this build does not have: use its shared-file method at every N
    cmd += ["-pn", str(world), "-pr", str(rank), "-pg", "8", "-pi", "fs", "-pf", sync_dir]
    env = dict(os.environ)
    if world > 1:
        env["CUDA_VISIBLE_DEVICES"] = env.get("CUDA_VISIBLE_DEVICES", ",".join(str(i) for i in range(8)))
    sampler = ClockSampler(local)
    sampler.start()
    t0 = time.perf_counter()
    try:
        res = subprocess.run(cmd, cwd=ref_dir, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=3000)
    except subprocess.TimeoutExpired:
        sampler.stop()
        return unavailable("the reference trainer did not finish within 3000 s")
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    if rank == 0:
        try:
            os.remove(os.path.join(sync_dir, "ready"))
        except OSError:
            pass
    if res.returncode != 0:
        tail = " | ".join(res.stdout.strip().splitlines()[-3:])
        return unavailable("the reference trainer exited with code %d: %s" % (res.returncode, tail[:300]))
    # rank 0 of the reference prints: step    4/10 | loss ... | 512.34 ms | ...% bf16 MFU | ... tok/s
    ms = [float(m.group(2)) for m in re.finditer(r"step\s+(\d+)/\d+ \|.*?\|\s+([0-9.]+) ms \|", res.stdout)]
    if world > 1:
        # only rank 0 prints; its step time is measured after the final device synchronisation of the step,
        # which follows the last collective, so it is the slowest rank's time
        if rank != 0:
            return 0
    if len(ms) < total_steps:
        return unavailable("could not parse %d step lines from the reference's output (got %d)" % (total_steps, len(ms)))
    timed = ms[a.warmup:a.warmup + a.steps]
    ms_per_step = sum(timed) / len(timed)
    value = a.total_batch / (ms_per_step / 1000.0)
    out = {
        "metric": metric_name(a.model), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": (value / PUBLISHED_BASELINE if a.model == "d12" else None), "dtype": "bf16",
        "data": "synthetic (seeded uniform-random uint16 tokens, random-init weights)",
        "config": config_record(a, world, a.zero),
        "comm_backend": "nccl",
        "timing": "the reference's own per-step cudaEvent time (train_gpt2.cu:1827-1856), H2D of tokens and loss read-back included",
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms_per_step, "h2d_bytes_per_step": (a.total_batch // world) * 2 * 4,
                "d2h_bytes_per_step": 8, "note": "the reference's step time already spans its H2D copies and loss read-back",
                "process_wall_s": wall},
        "impl": "reference",
    }
    print(json.dumps(out), flush=True)
    return 0


def main():
    a = parse()
    if a.impl == "reference":
        return run_reference(a)
    run_ours(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
