"""Data parallelism with optional ZeRO-1 optimizer-state sharding on flat buffers.

Sharding rule (kept equal to the reference so that state files are interchangeable, llmc/zero.cuh:496-507 and
train_gpt2.cu:977-1124 of the reference): for every parameter tensor, rank r owns the elements
[r*S/N, (r+1)*S/N) of EVERY layer slice of size S; the optimizer arrays (m, v, master) are laid out tensor-major,
tensor i starting at (sum of the sizes of the tensors before it)/N, holding L consecutive layer shards.

Step on N ranks:
  backward (last micro-step): as soon as layer l's gradients are final, they are reduced to their owners
      (mean over ranks) on a side stream, overlapping the rest of backward;
  norm^2 of the reduced gradients over the own shards, summed over ranks;
  AdamW on the own shards with the clip coefficient computed on the device;
  all-gather of the updated bf16 shards.
The communication is delegated to a backend object (``comm``): ``NcclBackend`` issues NCCL collectives and is
the measured baseline; ``P2PBackend`` (p2p.py) runs this library's own kernels over NVLink peer memory.
"""
import torch
import torch.distributed as dist

from .. import ops
from ..models.gpt2 import DECAYED
from ..utils.sampler import Sampler


class SingleBackend:
    """One process: nothing to communicate."""
    name = "single"

    def reduce_tensors(self, grads_flat, slices, stream_event=None, tail=False):
        pass

    def finish_reduce(self):
        pass

    def all_reduce_scalar_sum(self, t):
        return t

    def all_gather_slices(self, params_flat, slices):
        pass

    def host_float_sum(self, value):
        return float(value)

    def host_barrier(self):
        pass

    def end_step(self, updated):
        pass


class NcclBackend:
    """NCCL collectives on a side stream (the reference's scheme, llmc/zero.cuh:528-551)."""
    name = "nccl"

    def __init__(self, cfg, zero_stage):
        self.cfg, self.zero_stage = cfg, zero_stage
        self.N, self.r = cfg.num_processes, cfg.process_rank
        self.cuda = cfg.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=cfg.device) if self.cuda else None
        self.avg = dist.ReduceOp.AVG if self.cuda else dist.ReduceOp.SUM     # gloo has no AVG

    def reduce_tensors(self, grads_flat, slices, stream_event=None, tail=False):
        """slices: list of (offset, size) of whole per-layer tensors.  ZeRO-1: reduce-scatter in place (the owner's shard
        receives the mean); otherwise all-reduce."""
        def run():
            for off, size in slices:
                full = grads_flat[off:off + size]
                if self.zero_stage == 1:
                    sh = size // self.N
                    out = full[self.r * sh:(self.r + 1) * sh]
                    if self.cuda:
                        dist.reduce_scatter_tensor(out, full, op=self.avg)
                    else:                                   # gloo: no reduce_scatter; emulate
                        tmp = full.float()
                        dist.all_reduce(tmp)
                        out.copy_(tmp[self.r * sh:(self.r + 1) * sh] / self.N)
                else:
                    if self.cuda:
                        dist.all_reduce(full, op=self.avg)
                    else:
                        tmp = full.float()
                        dist.all_reduce(tmp)
                        full.copy_(tmp / self.N)
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                run()
        else:
            run()

    def finish_reduce(self):
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)

    def all_reduce_scalar_sum(self, t):
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t

    def host_float_sum(self, value):
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.cfg.device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def host_barrier(self):
        dist.barrier()

    def end_step(self, updated):
        pass

    def all_gather_slices(self, params_flat, slices):
        for off, size in slices:
            full = params_flat[off:off + size]
            sh = size // self.N
            if self.cuda:
                dist.all_gather_into_tensor(full, full[self.r * sh:(self.r + 1) * sh].clone())
            else:
                parts = [torch.empty(sh, dtype=full.dtype) for _ in range(self.N)]
                dist.all_gather(parts, full[self.r * sh:(self.r + 1) * sh].clone())
                full.copy_(torch.cat(parts))


class ShardedAdamW:
    def __init__(self, model, cfg, zero_stage=0, use_master_weights=True, backend=None, beta1=0.9, beta2=0.95, eps=1e-8,
                 grad_clip=1.0):
        self.model, self.cfg = model, cfg
        self.N, self.r = cfg.num_processes, cfg.process_rank
        if zero_stage not in (0, 1):
            print("ZeRO stage %d is not supported; falling back to stage 0" % zero_stage)
            zero_stage = 0
        sizes = model.tensor_sizes()
        if zero_stage == 1 and self.N > 1:
            if any(per % (self.N * 8) for _, _, per, _ in sizes):
                print("a parameter tensor is not divisible by 8 x number of processes; ZeRO-1 disabled")
                zero_stage = 0
        if self.N == 1:
            zero_stage = 0
        self.zero_stage = zero_stage
        self.sharded = zero_stage == 1
        self.use_master = use_master_weights and model.dtype != torch.float32
        self.beta1, self.beta2, self.eps, self.grad_clip = beta1, beta2, eps, grad_clip
        self.backend = backend if backend is not None else (SingleBackend() if self.N == 1 else NcclBackend(cfg, zero_stage))
        if hasattr(self.backend, "zero_stage") and self.backend.zero_stage != zero_stage:
            if getattr(self.backend, "name", "") == "p2p" and any(per % (self.N * 8) for _, _, per, _ in sizes):
                raise ValueError("the in-kernel NVLink backend needs every parameter tensor divisible by 8 x number of processes; use -cb nccl")
            self.backend.zero_stage = zero_stage
        div = self.N if self.sharded else 1
        self.shard_num_parameters = model.num_parameters // div
        dev = model.device
        # optimizer state falls back to managed memory when the device is full (utils/memory.py)
        from ..utils.memory import zeros_device_or_managed
        n = self.shard_num_parameters
        self.m, m_managed = zeros_device_or_managed(n, torch.float32, dev, "AdamW first moment")
        self.v, v_managed = zeros_device_or_managed(n, torch.float32, dev, "AdamW second moment")
        self.master, w_managed = zeros_device_or_managed(n, torch.float32, dev, "master weights") if self.use_master else (None, False)
        self.state_in_managed_memory = m_managed or v_managed or w_managed
        self.master_initialized = False
        # [0] squared gradient norm, [1] mean loss of the step summed over ranks: reduced over the ranks together, read back together
        self.scalars = torch.zeros(2, dtype=torch.float32, device=dev)
        self.norm_sq = self.scalars[0:1]
        # stochastic-rounding seed stream: per rank when every rank rounds its own shard (the reference's 13371337 + rank); the same
        # on every rank when all of them update full replicas, so that the replicas stay bit-identical
        self.sampler = Sampler(13371337 + (self.r if self.sharded else 0))
        self.rng_state_last_update = self.sampler.state.value
        # static part of the views
        self.base_views = []
        o = 0
        for name, off, per, L in sizes:
            n = per // div
            self.base_views.append(dict(name=name, p_base=off + (self.r * n if self.sharded else 0), p_stride=per, o_base=o,
                                        o_stride=n, n=n, L=L))
            o += n * L
        self.layer_slices = {}
        for name, off, per, L in sizes:
            for l in range(L):
                key = l if L > 1 else -1
                self.layer_slices.setdefault(key, []).append((off + l * per, per))
        model.grad_hook = self.on_layer_grads_ready

    # ---- gradient reduction, overlapped with backward
    def on_layer_grads_ready(self, layer):
        if self.N > 1:
            self.backend.reduce_tensors(self.model.grads_flat, self.layer_slices[layer], tail=(layer == -1))

    def views(self, weight_decay=0.0, seeds=None):
        out = []
        for i, b in enumerate(self.base_views):
            v = dict(b)
            v["wd"] = weight_decay if b["name"] in getattr(self.model, "decayed", DECAYED) else 0.0
            v["seed"] = seeds[i] if seeds is not None else 0
            out.append(v)
        return out

    def grad_norm_sq(self, loss_terms=None, loss_scale=1.0):
        """Device tensor holding the squared norm of the (reduced) gradient over all ranks.  With ``loss_terms`` (the per-token
        losses of this rank), ``self.scalars[1]`` receives loss_scale * sum(loss_terms) summed over the ranks in the same
        exchange (reference: the ncclAllReduce calls of train_gpt2.cu:958 and :1022), so that every rank sees the same loss."""
        if self.N > 1:
            self.backend.finish_reduce()
        if self.N > 1 and hasattr(self.backend, "fused_norm_sq"):
            # partial sums of squares were produced by the reduction kernels; one launch sums them, sums the losses and exchanges both
            self.backend.fused_norm_sq(self.scalars, loss_terms, loss_scale)
            return self.norm_sq
        ops.global_norm_sq(self.norm_sq, self.model.grads_flat, self.views())
        if loss_terms is not None:
            ops.sum_scaled(self.scalars[1:2], loss_terms, loss_scale)
        if self.N > 1:
            if self.sharded:
                self.backend.all_reduce_scalar_sum(self.scalars)
            elif loss_terms is not None:
                self.backend.all_reduce_scalar_sum(self.scalars[1:2])      # gradients are replicated: only the loss differs per rank
        return self.norm_sq

    def step(self, learning_rate, weight_decay, t, grad_scale=1.0, init_from_master_only=False):
        """One update; t counts from 1.  The clip coefficient min(1, clip/|g|) is applied on the device from
        ``self.norm_sq`` (call grad_norm_sq() first); a non-finite norm skips the update."""
        model = self.model
        self.rng_state_last_update = self.sampler.state.value
        seeds = [self.sampler.random_u32() for _ in self.base_views]
        views = self.views(weight_decay, seeds)
        fused = self.sharded and hasattr(self.backend, "adamw_allgather")
        if init_from_master_only:
            ops.params_from_master(model.params_flat, self.master, views)
            if fused:                                      # one-off at resume: gather through the process group
                NcclBackend(self.cfg, 1).all_gather_slices(model.params_flat, self._all_slices())
                return
        elif fused:
            if self.use_master and not self.master_initialized:
                ops.master_from_params(self.master, model.params_flat, views)
                self.master_initialized = True
            self.backend.adamw_allgather(self.master, self.m, self.v, views, learning_rate, self.beta1, self.beta2, self.eps, t,
                                         grad_scale, self.norm_sq, self.grad_clip)
            return
        else:
            if self.use_master and not self.master_initialized:
                ops.master_from_params(self.master, model.params_flat, views)
                self.master_initialized = True
            ops.adamw_update(model.params_flat, self.master, model.grads_flat, self.m, self.v, views, learning_rate, self.beta1,
                             self.beta2, self.eps, t, grad_scale, self.norm_sq, self.grad_clip)
        if self.sharded:
            self.backend.all_gather_slices(model.params_flat, self._all_slices())

    def sync_params(self):
        """Blocks the current stream until this rank's copy of the parameters is complete.  The forward pass does its own,
        finer-grained waiting; anything else that reads ``params_flat`` after a step (checkpoint writer, export) calls this."""
        if hasattr(self.backend, "wait_params"):
            self.backend.wait_params()

    def _all_slices(self):
        slices = []
        for name, off, per, L in self.model.tensor_sizes():
            slices += [(off + l * per, per) for l in range(L)]
        return slices
