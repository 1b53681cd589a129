"""Training entry point with the command-line surface of the reference's ``train_gpt2cu``
(train_gpt2.cu:1362-1903 of the reference): the same short flags, stdout step line, ``main.log``, checkpoint files,
resume logic, validation / HellaSwag / sampling cadence.

``Trainer`` is the public API: build one from ``TrainConfig`` (or ``parse_args``), then call ``train_step()`` per
optimizer step or ``run()`` for the whole loop.  A step enqueues all micro-steps, the gradient reduction, the norm,
the clip and the AdamW update without waiting for the GPU, and reads loss and gradient norm back once at the end.
"""
import glob as _glob
import ctypes
import math
import os
import sys
import time
from dataclasses import dataclass, field

import torch

from . import ops
from .models import gpt2, llama3
from .parallel import dist as pdist
from .parallel.zero import ShardedAdamW
from .utils import checkpoint, mfu
from .utils.dataloader import DataLoader, EvalLoader
from .utils.logger import Logger
from .utils.outlier import OutlierDetector
from .utils.sampler import Sampler
from .utils.schedulers import LearningRateScheduler
from .utils.tokenizer import Tokenizer, printable

USAGE = """Usage:   python train_gpt2.py [options]
Options (same letters as the reference trainer):
  -i <str>   train data filename pattern (default dev/data/tinyshakespeare/tiny_shakespeare_train.bin)
  -j <str>   val data filename pattern
  -e <str>   model checkpoint .bin (GPT-2/3 or LLaMA-3 file), or a descriptor dN | gpt2:dN | gpt3:cN | llama3:8B | llama3:l=..,c=..
             for random init (default gpt2_124M_bf16.bin)
  -lg <int>  log GPU telemetry every N steps (default -1: never)
  -o <str>   output log dir (default: none, no logging / checkpoints)
  -n <int>   write checkpoints every N steps (default 0: never)   -nk <int> keep the last K   -nm <int> never delete multiples of M
  -y <int>   resume from the latest checkpoint in the output dir (default 0)
  -b <int>   micro batch size per GPU (default 4)     -t <int> sequence length (default 1024)
  -d <int>   total batch size in tokens (default B*T*num_processes)
  -x <int>   max steps (default -1: one epoch)
  -k <str>   lr scheduler cosine|linear|constant|wsd   -l <float> learning rate (3e-4)   -u <int> warmup iters (0)
  -q <float> final lr fraction (1.0)   -c <float> weight decay (0.0)
  -sl <float> skip update if loss z-score above (0 = off)   -sg <float> same for the gradient norm
  -v <int> val_loss_every (20)  -m <int> val_max_steps (20)  -s <int> sample_every (20)  -g <int> genT (64)  -h <int> HellaSwag eval (0)
  -a <int> overfit a single batch (0)
  -f <int> TF32 matmuls in the fp32 device mode (1)   -w <int> fp32 master weights (1)   -ge <int> GELU fusion (accepted)
  -z <int> ZeRO stage 0|1 (0)   -r <int> recompute 0|1|2 (1)
  -pn <int> num processes  -pr <int> process rank  -pg <int> GPUs per node  -pi <str> init method mpi|tcp|fs  -ps <ip>  -pf <path>
Extensions:  -dev cpu|cuda   -dt bf16|fp32   -cb nccl|p2p (communication backend of the multi-GPU step)
             -b2 <float> AdamW beta2 (0.95)   -gc <float> gradient clipping norm (1.0; 0 = off)   -hp / -tp HellaSwag / tokenizer paths
             -fw <float> limit, in seconds, of a kernel's wait for a flag written by another GPU (0 = the library's default, about 10 s)
             -wd <float> watchdog: end the process (exit code 17) if no optimizer step completes within this many seconds (0 = off)
"""


@dataclass
class TrainConfig:
    train_data_pattern: str = "dev/data/tinyshakespeare/tiny_shakespeare_train.bin"
    val_data_pattern: str = "dev/data/tinyshakespeare/tiny_shakespeare_val.bin"
    load_filename: str = "gpt2_124M_bf16.bin"
    lr_scheduler_type: str = "cosine"
    output_log_dir: str = ""
    checkpoint_every: int = 0
    checkpoints_keep: int = 0
    major_checkpoint_every: int = 0
    resume: int = 0
    B: int = 4
    T: int = 1024
    total_batch_size: int = -1
    learning_rate: float = 3e-4
    log_gpu_every: int = -1
    warmup_iterations: int = 0
    final_learning_rate_frac: float = 1.0
    weight_decay: float = 0.0
    skip_update_lossz: float = 0.0
    skip_update_gradz: float = 0.0
    val_loss_every: int = 20
    val_max_steps: int = 20
    sample_every: int = 20
    genT: int = 64
    overfit_single_batch: int = 0
    max_steps: int = -1
    override_enable_tf32: int = 1
    use_master_weights: int = 1
    gelu_fusion: int = -1
    recompute: int = 1
    zero_stage: int = 0
    hellaswag_eval: int = 0
    num_processes: int = 1
    process_rank: int = 0
    gpus_per_node: int = 8
    nccl_init_method: str = "mpi"
    server_ip: str = ""
    fs_path: str = ""
    device: str = ""
    dtype: str = ""
    comm_backend: str = ""
    hellaswag_path: str = "dev/data/hellaswag/hellaswag_val.bin"
    tokenizer_path: str = "gpt2_tokenizer.bin"
    quiet: bool = False
    prefetch: bool = True
    beta2: float = 0.95
    grad_clip: float = 1.0
    flag_wait_s: float = 0.0      # > 0: limit of in-kernel waits for peer flags, in seconds
    watchdog_s: float = 0.0       # > 0: end the process if no optimizer step completes within this many seconds


_FLAGS = {
    "-i": ("train_data_pattern", str), "-j": ("val_data_pattern", str), "-e": ("load_filename", str), "-o": ("output_log_dir", str),
    "-k": ("lr_scheduler_type", str), "-n": ("checkpoint_every", int), "-nk": ("checkpoints_keep", int),
    "-nm": ("major_checkpoint_every", int), "-y": ("resume", int), "-b": ("B", int), "-t": ("T", int), "-d": ("total_batch_size", int),
    "-l": ("learning_rate", float), "-lg": ("log_gpu_every", int), "-u": ("warmup_iterations", int),
    "-q": ("final_learning_rate_frac", float), "-c": ("weight_decay", float), "-x": ("max_steps", int), "-v": ("val_loss_every", int),
    "-m": ("val_max_steps", int), "-s": ("sample_every", int), "-g": ("genT", int), "-h": ("hellaswag_eval", int),
    "-a": ("overfit_single_batch", int), "-f": ("override_enable_tf32", int), "-w": ("use_master_weights", int),
    "-ge": ("gelu_fusion", int), "-z": ("zero_stage", int), "-r": ("recompute", int), "-pn": ("num_processes", int),
    "-pr": ("process_rank", int), "-pg": ("gpus_per_node", int), "-pi": ("nccl_init_method", str), "-pm": ("nccl_init_method", str),
    "-ps": ("server_ip", str), "-pf": ("fs_path", str), "-pp": ("fs_path", str), "-sl": ("skip_update_lossz", float),
    "-sg": ("skip_update_gradz", float), "-dev": ("device", str), "-dt": ("dtype", str), "-cb": ("comm_backend", str),
    "-hp": ("hellaswag_path", str), "-tp": ("tokenizer_path", str), "-b2": ("beta2", float), "-gc": ("grad_clip", float),
    "-wd": ("watchdog_s", float),
    "-fw": ("flag_wait_s", float),
}


class UsageError(Exception):
    pass


def parse_args(argv):
    """Pairs of ``-flag value`` exactly like the reference's parser (train_gpt2.cu:1459-1502)."""
    cfg = TrainConfig()
    if len(argv) % 2 != 0:
        raise UsageError("flags come in pairs: -flag value")
    for i in range(0, len(argv), 2):
        flag, val = argv[i], argv[i + 1]
        if not flag.startswith("-") or flag not in _FLAGS:
            raise UsageError("unknown flag %s" % flag)
        name, typ = _FLAGS[flag]
        try:
            setattr(cfg, name, typ(val))
        except ValueError:
            raise UsageError("bad value %r for %s" % (val, flag))
    return cfg


class Trainer:
    def __init__(self, cfg, dist_cfg=None):
        self.cfg = cfg
        c = cfg
        device_type = c.device or None
        self.dist = dist_cfg or pdist.init_distributed(c.num_processes, c.process_rank, c.gpus_per_node, c.nccl_init_method,
                                                       c.server_ip, c.fs_path, device_type)
        d = self.dist
        self.device = d.device
        self.print0 = (lambda *a, **k: print(*a, **k, flush=True)) if (d.is_main and not c.quiet) else (lambda *a, **k: None)
        dtype = {"": None, "bf16": torch.bfloat16, "fp32": torch.float32}[c.dtype]
        B, T = c.B, c.T
        tokens_per_fwdbwd = B * T * d.num_processes
        if c.total_batch_size == -1:
            c.total_batch_size = tokens_per_fwdbwd
        if c.total_batch_size % tokens_per_fwdbwd != 0:
            raise ValueError("total batch size %d is not a multiple of B*T*num_processes = %d" % (c.total_batch_size, tokens_per_fwdbwd))
        self.grad_accum_steps = c.total_batch_size // tokens_per_fwdbwd
        if c.gelu_fusion == -1:
            c.gelu_fusion = 2

        # ---- model: resume > checkpoint file > descriptor
        self.resuming = False
        self.resume_step = -1
        if c.resume == 1 and c.output_log_dir:
            self.resume_step = checkpoint.find_max_step(c.output_log_dir)
            self.resuming = self.resume_step != -1
        load = c.load_filename
        if self.resuming:
            load = checkpoint.checkpoint_paths(c.output_log_dir, self.resume_step, d.process_rank)[0]
        # multi-GPU ZeRO-1 on this library's own NVLink kernels: the flat buffers live in symmetric memory
        arena, sym_bufs, allocator = None, {}, None
        if d.num_processes > 1 and self.device.type == "cuda" and dtype != torch.float32 and (c.comm_backend or "p2p") == "p2p":
            from .parallel import p2p
            arena = p2p.try_create(None, d, c.zero_stage, self.print0)
            if arena is not None:
                def allocator(kind, numel, dt):
                    sym_bufs[kind] = arena.alloc(numel, dt)
                    return sym_bufs[kind][0]
        if load.endswith(".bin"):
            mcfg, _ = checkpoint.read_model_header(load)
            cls = llama3.Llama if checkpoint.model_family(load) == "llama3" else gpt2.GPT
            self.model = cls(mcfg, self.device, dtype, recompute=c.recompute, flat_allocator=allocator)
            checkpoint.load_model(load, self.model)
        elif load.startswith("llama3:"):
            self.model = llama3.Llama(llama3.config_from_descriptor(load), self.device, dtype, recompute=c.recompute,
                                      flat_allocator=allocator)
            self.model.init_random(42)
        else:
            self.model = gpt2.GPT(gpt2.config_from_descriptor(load), self.device, dtype, recompute=c.recompute, flat_allocator=allocator)
            self.model.init_random(42)
        m = self.model
        if T > m.cfg.max_seq_len:
            raise ValueError("sequence length %d exceeds the model's maximum %d" % (T, m.cfg.max_seq_len))
        self.precision = "bf16" if m.dtype == torch.bfloat16 else "fp32"
        if self.device.type == "cuda" and m.dtype == torch.float32:
            # full-precision mode: -f 1 lets the library GEMMs use TF32 tensor cores, -f 0 keeps them in IEEE fp32
            # (the same switch as the reference's train_gpt2_fp32.cu / PRECISION=FP32 builds)
            torch.backends.cuda.matmul.allow_tf32 = bool(c.override_enable_tf32)

        # ---- data
        permute = 0 if c.overfit_single_batch == 1 else 1
        self.train_loader = DataLoader(c.train_data_pattern, B, T, d.process_rank, d.num_processes, permute, prefetch=c.prefetch)
        self.val_loader = DataLoader(c.val_data_pattern, B, T, d.process_rank, d.num_processes, 0) if c.val_data_pattern else None
        self.train_num_batches = self.train_loader.num_tokens // c.total_batch_size
        if c.max_steps > -1:
            self.train_num_batches = c.max_steps
        self.val_num_batches = 0
        if self.val_loader is not None:
            self.val_num_batches = self.val_loader.num_tokens // tokens_per_fwdbwd
            if c.val_max_steps >= 0:
                self.val_num_batches = min(self.val_num_batches, c.val_max_steps)
        self.eval_loader = None
        if c.hellaswag_eval and os.path.exists(c.hellaswag_path) and B >= 4:
            self.eval_loader = EvalLoader(c.hellaswag_path, B, T, d.process_rank, d.num_processes)

        # ---- optimizer / parallel
        backend = None
        m.allocate_grads()
        if arena is not None:
            from .parallel import p2p
            backend = p2p.P2PBackend(m, d, arena, sym_bufs["params"], sym_bufs["grads"], zero_stage=(1 if c.zero_stage == 1 else 0))
        self.opt = ShardedAdamW(m, d, c.zero_stage, bool(c.use_master_weights), backend, beta2=c.beta2,
                                grad_clip=(c.grad_clip if c.grad_clip > 0 else 1e30))
        if c.flag_wait_s > 0 and self.device.type == "cuda":
            # the limit is counted in SM clock cycles; 2 GHz is an upper bound of the clock, so the wait lasts at least flag_wait_s
            from . import _lib
            _lib.check(_lib.cuda().llmc_p2p_set_wait_cycles(ctypes.c_longlong(int(c.flag_wait_s * 2.0e9))), "llmc_p2p_set_wait_cycles")
        self.logger = Logger(c.output_log_dir, d.process_rank, self.resuming)
        self.tokenizer = Tokenizer(c.tokenizer_path)
        self.scheduler = LearningRateScheduler(c.lr_scheduler_type, c.learning_rate, c.warmup_iterations, self.train_num_batches,
                                               c.final_learning_rate_frac)
        self.loss_detector, self.norm_detector = OutlierDetector(), OutlierDetector()
        self.sample_rng = Sampler(1337)
        self.step = 0
        self.ema_tokens_per_second = 0.0
        self.telemetry = None
        self._h2d_events = None
        self._sample_model = None
        self._sample_gen = None
        self._have_batch = False
        self._measured_peak = None
        from .utils.watchdog import StepWatchdog
        self.watchdog = StepWatchdog(c.output_log_dir, d.process_rank, d.num_processes, c.watchdog_s).start()
        m.allocate_activations(B, T)
        if self.device.type == "cuda":
            self._h2d_events = [torch.cuda.Event(), torch.cuda.Event()]
            for ev in self._h2d_events:
                ev.record()
            # a pinned batch buffer may be refilled only after its host-to-device copy has run
            self.train_loader.before_fill = lambda i: self._h2d_events[i].synchronize()
            self.device_name = torch.cuda.get_device_name(self.device)
        else:
            self.device_name = "cpu"
        if self.resuming:
            self._load_state()
        self._print_header()

    # ------------------------------------------------------------------ reporting
    def _print_header(self):
        c, m, d = self.cfg, self.model, self.dist
        p = self.print0
        p("+-----------------------+----------------------------------------------------+")
        p("| Parameter             | Value                                              |")
        p("+-----------------------+----------------------------------------------------+")
        rows = [("train data pattern", c.train_data_pattern), ("val data pattern", c.val_data_pattern), ("output log dir", c.output_log_dir or "NULL"),
                ("checkpoint_every", c.checkpoint_every), ("resume", c.resume), ("micro batch size B", c.B), ("sequence length T", c.T),
                ("total batch size", c.total_batch_size), ("LR scheduler", c.lr_scheduler_type), ("learning rate (LR)", "%e" % c.learning_rate),
                ("warmup iterations", c.warmup_iterations), ("final LR fraction", "%e" % c.final_learning_rate_frac), ("weight decay", "%e" % c.weight_decay),
                ("skip update lossz", c.skip_update_lossz), ("skip update gradz", c.skip_update_gradz), ("max_steps", c.max_steps),
                ("val_loss_every", c.val_loss_every), ("val_max_steps", c.val_max_steps), ("sample_every", c.sample_every), ("genT", c.genT),
                ("overfit_single_batch", c.overfit_single_batch), ("use_master_weights", "enabled" if self.opt.use_master else "disabled"),
                ("gelu_fusion", c.gelu_fusion), ("recompute", c.recompute), ("device", self.device_name), ("precision", self.precision.upper()),
                ("load_filename", c.load_filename), ("max_sequence_length T", m.cfg.max_seq_len), ("vocab_size V", m.cfg.vocab_size),
                ("padded_vocab_size Vp", m.cfg.padded_vocab_size), ("num_layers L", m.cfg.num_layers), ("num_heads NH", m.cfg.num_heads),
                ("channels C", m.cfg.channels), ("num_parameters", m.num_parameters), ("train_num_batches", self.train_num_batches),
                ("val_num_batches", self.val_num_batches), ("num_processes", d.num_processes), ("zero_stage", self.opt.zero_stage),
                ("comm backend", self.opt.backend.name), ("grad_accum_steps", self.grad_accum_steps)]
        for k, v in rows:
            p("| %-21s | %-50s |" % (k, v))
        p("+-----------------------+----------------------------------------------------+")
        p("allocated %d MiB for activations, %d MiB for parameters, %d MiB for AdamW state shards" % (
            m.activation_bytes() >> 20, (m.params_flat.numel() * m.params_flat.element_size()) >> 20,
            (self.opt.m.numel() * 4 * (3 if self.opt.use_master else 2)) >> 20))

    # ------------------------------------------------------------------ state
    def _load_state(self):
        c, d = self.cfg, self.dist
        _, state_path, _ = checkpoint.checkpoint_paths(c.output_log_dir, self.resume_step, d.process_rank)
        info = checkpoint.read_state(state_path, num_processes=d.num_processes, process_rank=d.process_rank, m=self.opt.m, v=self.opt.v,
                                     master=self.opt.master, loader=self.train_loader)
        self.step = info["step"]
        self.opt.master_initialized = True
        if self.opt.use_master and info["use_master_weights"]:
            # re-round the bf16 parameters from the master copy with the seeds of the last update: bit-identical parameters
            self.opt.sampler.state.value = info["rng_state_last_update"]
            self.opt.step(0.0, 0.0, 1, init_from_master_only=True)
        self.opt.sampler.state.value = info["rng_state"]
        self.opt.rng_state_last_update = info["rng_state_last_update"]

    def write_checkpoint(self, step):
        c, d = self.cfg, self.dist
        model_path, state_path, done_path = checkpoint.checkpoint_paths(c.output_log_dir, step, d.process_rank)
        self.print0("Writing model to %s" % model_path)
        self.opt.sync_params()                      # every rank's shards of the last update have landed in this rank's copy
        if d.is_main:
            checkpoint.write_model(model_path, self.model)
        checkpoint.write_state(state_path, num_processes=d.num_processes, process_rank=d.process_rank, use_master_weights=self.opt.use_master,
                               step=step, rng_state=self.opt.sampler.state.value, rng_state_last_update=self.opt.rng_state_last_update,
                               m=self.opt.m, v=self.opt.v, master=self.opt.master, loader=self.train_loader)
        self.opt.backend.host_barrier()             # every rank's state file is complete before the marker appears
        if d.is_main:
            open(done_path, "w").close()

    # ------------------------------------------------------------------ evaluation helpers
    def _upload(self, inputs, targets, buf_index=None):
        m = self.model
        # token ids index the embedding table on the device: refuse a corrupt batch on the host (reference: tokenCheck)
        hi = max(int(inputs.max()), int(targets.max()))
        lo = min(int(inputs.min()), int(targets.min()))
        if lo < 0 or hi >= m.cfg.vocab_size:
            raise ValueError("token id out of range [0, %d): got %d / %d" % (m.cfg.vocab_size, lo, hi))
        m.inputs.copy_(inputs, non_blocking=True)
        m.targets.copy_(targets, non_blocking=True)
        if self._h2d_events is not None and buf_index is not None:
            self._h2d_events[buf_index].record()

    def validate(self):
        m, vl = self.model, self.val_loader
        vl.reset()
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        for _ in range(self.val_num_batches):
            inputs, targets = vl.next_batch()
            self._upload(inputs, targets)
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()      # the pinned buffers are reused by the next batch
            m.forward(m.inputs, m.targets, 1, 0, write_dlogits=False)
            total += m.loss(1)
        val = float(total.item()) / max(self.val_num_batches, 1)
        return self.opt.backend.host_float_sum(val) / self.dist.num_processes

    def hellaswag(self):
        m, el = self.model, self.eval_loader
        el.reset()
        correct = 0
        for _ in range(el.num_batches):
            inputs, targets, _mask = el.next_batch()
            self._upload(inputs, targets)
            m.forward(m.inputs, m.targets, 1, 0, write_dlogits=False)
            correct += el.stat_losses(m.acts["losses"].view(self.cfg.B, self.cfg.T))
        total = self.opt.backend.host_float_sum(correct)
        return total / el.num_examples

    def sample(self, genT):
        """Autoregressive sampling on rank 0 (full prefix recomputed per token, as in the reference train_gpt2.cu:1752-1796)."""
        m = self.model
        if getattr(m, "family", "") == "llama3":
            # key / value cache, nucleus sampling at the reference script's settings (train_llama3.py:1172)
            from .models.generate import generate
            if self._sample_gen is None:
                self._sample_gen = torch.Generator().manual_seed(1337)
            start = min(128000, m.cfg.vocab_size - 1)                       # <|begin_of_text|>
            stops = [t for t in (128001, 128009) if t < m.cfg.vocab_size]   # <|end_of_text|>, <|eot_id|>
            return generate(m, [[start]], max(genT - 1, 1), temperature=0.6, top_p=0.9, stop_tokens=stops, generator=self._sample_gen)[0]
        if self._sample_model is None:
            # a second model object over the same parameter buffer, with its own (small) activation set
            sm = type(m)(m.cfg, self.device, m.dtype, recompute=2, flat_allocator=lambda kind, numel, dt: m.params_flat)
            sm.param_sync = m.param_sync
            self._sample_model = sm
        sm = self._sample_model
        eot = min(self.tokenizer.eot_token, m.cfg.vocab_size - 1)
        Tmax = min(m.cfg.max_seq_len, max(genT, 1))
        chunk = min(self.cfg.T, 256)
        tokens = torch.full((1, Tmax), eot, dtype=torch.int32)
        out = []
        for t in range(1, min(genT, m.cfg.max_seq_len + 1)):      # the context window bounds the generation
            Tcur = min(m.cfg.max_seq_len, -(-t // chunk) * chunk)
            dev_tokens = torch.full((1, Tcur), eot, dtype=torch.int32)
            dev_tokens[0, :min(t, Tcur)] = tokens[0, :min(t, Tcur)]
            sm.forward(dev_tokens.to(self.device))
            logits = sm.logits()[0, t - 1, :m.cfg.vocab_size].float().cpu()
            nxt = self.sample_rng.sample_softmax(logits)
            if t < Tmax:
                tokens[0, t] = nxt
            out.append(nxt)
        return out

    # ------------------------------------------------------------------ the step
    def train_step(self):
        """One optimizer step.  Returns dict(loss, grad_norm, lr, skipped).  One device synchronisation, at the end."""
        c, m, opt = self.cfg, self.model, self.opt
        tl = self.train_loader
        step = self.step
        G = self.grad_accum_steps
        for micro in range(G):
            if c.overfit_single_batch == 0 or not self._have_batch:
                inputs, targets = tl.next_batch()
                self._upload(inputs, targets, tl.last_index)
                self._have_batch = True
            m.forward(m.inputs, m.targets, G, micro)
            m.backward(micro, last_micro_step=(micro == G - 1))
        # the squared gradient norm and the mean loss are summed over the ranks in one exchange and read back in one copy; every
        # rank sees the same two numbers, so every rank takes the same decision about skipping the update
        B_, T_ = m.act_shape
        opt.grad_norm_sq(m.acts["losses"], 1.0 / float(B_ * T_ * G))
        lr = self.scheduler.get_learning_rate(step)
        nproc = self.dist.num_processes

        def read_back():
            vals = opt.scalars.cpu()                                              # the single synchronisation of the step
            nsq = float(vals[0])
            return float(vals[1]) / nproc, (math.sqrt(max(nsq, 0.0)) if math.isfinite(nsq) else float("nan"))

        need_host_decision = c.skip_update_lossz != 0.0 or c.skip_update_gradz != 0.0
        skipped = False
        if need_host_decision:
            loss, gnorm = read_back()
            zl, zg = self.loss_detector.update(loss), self.norm_detector.update(gnorm)
            if math.isfinite(zl) and c.skip_update_lossz != 0.0 and zl > c.skip_update_lossz:
                self.print0("skipping update due to loss z-score of %f" % zl)
                skipped = True
            elif math.isfinite(zg) and c.skip_update_gradz != 0.0 and zg > c.skip_update_gradz:
                self.print0("skipping update due to grad z-score of %f" % zg)
                skipped = True
            if not skipped:
                opt.step(lr, c.weight_decay, step + 1)
        else:
            opt.step(lr, c.weight_decay, step + 1)
            loss, gnorm = read_back()
            zl, zg = self.loss_detector.update(loss), self.norm_detector.update(gnorm)
        opt.backend.end_step(updated=not skipped)
        if self.device.type == "cuda":
            # a kernel that gave up a bounded wait (peer flag, mbarrier) left its reason in the status word; the device is
            # idle here (the loss was just read back), so reading it costs one small copy
            from . import _lib
            status = _lib.read_status(clear=True)
            if status != 0:
                raise RuntimeError("a kernel reported an abandoned wait: status 0x%08x (code %d at 0x%x) in step %d on rank %d"
                                   % (status, status >> 24, status & 0xFFFFFF, step, self.dist.process_rank))
        self.step += 1
        if self.watchdog.timeout_s > 0 or self.watchdog.log_dir:
            self.watchdog.beat(self.step)
        return dict(loss=loss, grad_norm=gnorm, lr=lr, skipped=skipped, zloss=zl, zgrad=zg)

    # ------------------------------------------------------------------ the loop
    def run(self):
        c, d = self.cfg, self.dist
        p = self.print0
        start_step = self.step
        beat = (lambda phase: self.watchdog.beat(self.step, phase)) if (self.watchdog.timeout_s > 0 or self.watchdog.log_dir) else (lambda phase: None)
        for step in range(start_step, self.train_num_batches + 1):
            last_step = step == self.train_num_batches
            # the first iteration of a resumed run does not rewrite the checkpoint it has just loaded: that one is complete and
            # carries its DONE marker, and a kill during the rewrite would leave a marked but damaged checkpoint
            # (reference: the `resuming == 0` guard of train_gpt2.cu:1799-1812)
            just_resumed = self.resuming and step == start_step
            if self.val_loader is not None and c.val_loss_every > 0 and (step % c.val_loss_every == 0 or last_step):
                beat("validation")
                val_loss = self.validate()
                p("val loss %f" % val_loss)
                self.logger.log_val(step, val_loss)
            if self.eval_loader is not None and ((step > 0 and step % c.val_loss_every == 0) or last_step):
                beat("evaluation")
                acc = self.hellaswag()
                p("HellaSwag: %.4f" % acc)
                self.logger.log_eval(step, acc)
            if c.sample_every > 0 and ((step > 0 and step % c.sample_every == 0) or last_step):
                beat("sampling")                      # every rank: only rank 0 samples, the others wait for it in their next step
            if d.is_main and c.sample_every > 0 and ((step > 0 and step % c.sample_every == 0) or last_step):
                toks = self.sample(c.genT)
                p("generating:\n---")
                if self.tokenizer.init_ok:
                    p("".join(printable(self.tokenizer.decode(t)) for t in toks))
                else:
                    p(" ".join(str(t) for t in toks))
                p("---")
            if c.output_log_dir and c.checkpoint_every > 0 and not just_resumed and ((step > 0 and step % c.checkpoint_every == 0) or last_step):
                beat("checkpoint")
                self.write_checkpoint(step)
                beat("checkpoint written")
                step_delete = step - c.checkpoints_keep * c.checkpoint_every
                if c.checkpoints_keep > 0 and step_delete > 0 and (c.major_checkpoint_every == 0 or step_delete % c.major_checkpoint_every != 0):
                    checkpoint.delete_checkpoint(c.output_log_dir, step_delete, d.process_rank)
            if last_step:
                break
            t0 = time.perf_counter()
            r = self.train_step()
            dt = time.perf_counter() - t0
            tokens = c.total_batch_size
            if step > start_step:                     # the first step pays for warm-up: keep it out of the average
                tps = tokens / dt
                self.ema_tokens_per_second = tps if self.ema_tokens_per_second == 0.0 else 0.95 * self.ema_tokens_per_second + 0.05 * tps
            mfu_v = mfu.estimate_mfu(self.model.flops_per_token(c.T), tokens // d.num_processes, dt, self.device_name, self.precision)
            # the MFU column is against the data-sheet peak of the device (2250 dense bf16 TFLOP/s on a B200), as the reference
            # prints it; the JSONL metrics also carry the fraction of the measured sustained matmul peak of this machine class
            p("step %4d/%d | loss %7.6f (%+.2fz)| norm %6.4f (%+.2fz)| lr %.2e | %.2f ms | %.1f%% %s MFU | %.0f tok/s" % (
                step + 1, self.train_num_batches, r["loss"], r["zloss"], r["grad_norm"], r["zgrad"], r["lr"], dt * 1000.0, 100.0 * mfu_v,
                self.precision, self.ema_tokens_per_second))
            if c.log_gpu_every > 0 and (step + 1) % c.log_gpu_every == 0:
                if self.telemetry is None:
                    self.telemetry = mfu.GPUTelemetry(d.local_device_idx)
                p(mfu.GPUTelemetry.format(self.telemetry.read()))
            self.logger.log_train(step, r["loss"], r["lr"], r["grad_norm"])
            if self._measured_peak is None:
                self._measured_peak = mfu.measured_peak_tflops()
            mfu_measured = (self.model.flops_per_token(c.T) * (tokens // d.num_processes) / dt / (self._measured_peak * 1e12)
                            if self._measured_peak > 0 and self.precision == "bf16" else -1.0)
            self.logger.log_metrics(step=step, loss=r["loss"], grad_norm=r["grad_norm"], lr=r["lr"], ms=dt * 1000.0, mfu=mfu_v,
                                    mfu_of_measured_peak=mfu_measured)
        p("total average iteration speed: %.0f tok/s (EMA)" % self.ema_tokens_per_second)

    def close(self):
        self.watchdog.stop()
        for l in (self.train_loader, self.val_loader, self.eval_loader):
            if l is not None:
                l.close()
        pdist.shutdown(self.dist)


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    try:
        cfg = parse_args(argv)
    except UsageError as e:
        print("error: %s\n%s" % (e, USAGE), file=sys.stderr)
        return 1
    trainer = Trainer(cfg)
    try:
        trainer.run()
    finally:
        trainer.close()
    return 0
