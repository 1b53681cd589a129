"""ZeRO-1 communication backend that runs this library's own kernels over NVLink peer memory (csrc/comm.cu).

The flat parameter and gradient buffers and one small signal buffer are allocated as symmetric memory
(``torch.distributed._symmetric_memory``: same size on every rank, every rank can address every peer's copy).
NCCL is used only to rendezvous and to exchange the buffer handles.  After that a training step issues no NCCL
call: the per-layer gradient reduce-scatter (fused with the 1/N scale and the norm^2 partial sums) or, without
optimizer-state sharding (-z 0), the all-reduce form of the same kernel; the one-shot all-reduce that carries the
squared norm and the loss together; the AdamW update fused with the all-gather of the rounded bf16 parameters;
host scalars (validation loss, evaluation counts) and the barrier before a checkpoint's DONE marker are all kernels
that load from / store to peer memory directly.

Capability parity: multi_gpu_async_reduce_gradient, the ncclAllReduce calls of the loss and the norm, the
ncclAllGather of gpt2_update, multi_gpu_cpu_float_sum and multi_gpu_barrier in the reference (llmc/zero.cuh:480-487,
528-551 and 582-594, train_gpt2.cu:958, 1002-1030 and 1101-1120).
"""
import ctypes
import os

import torch
import torch.distributed as dist

from .. import _lib
from .._lib import check
from ..ops import kernels

MAX_RANKS = 8
_configured = False


def _cfg_lib():
    global _configured
    lib = _lib.cuda()
    if not _configured:
        P, I, LL, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong
        lib.llmc_p2p_signal_words.restype = I
        lib.llmc_p2p_reduce_scatter.restype = I
        lib.llmc_p2p_reduce_scatter.argtypes = [P, P, P, P, I, I, I, I, U, P, I, I, I, P, P]
        lib.llmc_p2p_allreduce_scalar.restype = I
        lib.llmc_p2p_allreduce_scalar.argtypes = [P, P, I, I, U, P]
        lib.llmc_p2p_allreduce_scalars.restype = I
        lib.llmc_p2p_allreduce_scalars.argtypes = [P, P, I, P, I, P, I, F, I, I, U, P]
        lib.llmc_p2p_wait_range.restype = I
        lib.llmc_p2p_wait_range.argtypes = [P, I, I, I, I, I, U, P]
        lib.llmc_p2p_adamw_allgather.restype = I
        lib.llmc_p2p_adamw_allgather.argtypes = [P, P, P, P, P, P, ctypes.POINTER(_lib.TensorTable), I, I, F, F, F, F, I, F, P, F, U, P, I, I, P]
        lib.llmc_p2p_wait.restype = I
        lib.llmc_p2p_wait.argtypes = [P, I, I, I, I, U, P]
        lib.llmc_p2p_rs_partials.restype = I
        lib.llmc_p2p_rs_partials.argtypes = [I]
        lib.llmc_p2p_ag_flag_offset.restype = I
        lib.llmc_p2p_ag_flag_offset.argtypes = [I]
        lib.llmc_p2p_barrier.restype = I
        lib.llmc_p2p_barrier.argtypes = [P, I, I, U, P]
        lib.llmc_p2p_rs_handshake.restype = I
        lib.llmc_p2p_rs_handshake.argtypes = [P, I, I, I, U, P]
        _configured = True
    return lib


def _ptr_array(ptrs):
    return (ctypes.c_ulonglong * len(ptrs))(*[int(p) for p in ptrs])


class SymmetricArena:
    """Allocates tensors that every rank of the group can address on every peer."""

    def __init__(self, dist_cfg):
        import torch.distributed._symmetric_memory as symm
        self.symm = symm
        self.cfg = dist_cfg
        self.group = dist.group.WORLD
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")            # newer PyTorch enables every group by itself and only warns here
            try:
                symm.enable_symm_mem_for_group(self.group.group_name)
            except Exception:
                pass

    def alloc(self, numel, dtype, zero=True):
        t = self.symm.empty(int(numel), dtype=dtype, device=self.cfg.device)
        if zero:
            t.zero_()
        handle = self.symm.rendezvous(t, self.group.group_name)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        return t, ptrs, handle


class _Ready:
    """What a GEMM needs to wait for a parameter group inside the kernel: address of the N flags, N, the sequence number."""

    def __init__(self, backend, channel):
        self.backend, self.channel = backend, channel
        self.flags_ptr, self.n, self.seq = backend.flag_address(channel), backend.N, backend.published_seq

    def wait(self):
        self.backend.wait_params(self.channel)


class ParamSync:
    """The forward pass's view of parameters that may still be arriving from the other ranks.  ``wait(-1)`` precedes the first
    read of the shared group (embeddings, norms, LM head); ``flags(l)`` goes to the first GEMM of layer l, which polls inside
    the kernel."""

    def __init__(self, backend):
        self.backend = backend

    def wait(self, layer):
        self.backend.wait_params(layer + 1)

    def wait_all(self):
        """Every group, for readers outside the training forward pass (generation, checkpoints)."""
        self.backend.wait_params()

    def flags(self, layer):
        if self.backend.published_seq == 0:
            return None
        return _Ready(self.backend, layer + 1)


class P2PBackend:
    name = "p2p"

    def __init__(self, model, dist_cfg, arena, params, grads, zero_stage=1):
        self.cfg = dist_cfg
        self.zero_stage = zero_stage
        self.N, self.r = dist_cfg.num_processes, dist_cfg.process_rank
        self.lib = _cfg_lib()
        self.model = model
        self.params_t, self.param_ptrs, self._ph = params
        self.grads_t, self.grad_ptrs, self._gh = grads
        words = self.lib.llmc_p2p_signal_words()
        self.sig_t, self.sig_ptrs, self._sh = arena.alloc(words, torch.int64)
        self.c_params, self.c_grads, self.c_sig = _ptr_array(self.param_ptrs), _ptr_array(self.grad_ptrs), _ptr_array(self.sig_ptrs)
        dev = dist_cfg.device
        # LLMC_RS_PRIORITY=-1 makes the communication stream a high-priority stream (its CTAs are placed first when SMs free up)
        self.stream = torch.cuda.Stream(device=dev, priority=int(os.environ.get("LLMC_RS_PRIORITY", "0")))
        self.ctas = 32                  # x 4 = CTAs of the fused update + gather, which runs alone after backward
        # reduce-scatter: 32 whole-SM CTAs next to the backward pass (LLMC_RS_THREADS=128: one small CTA per SM instead)
        self.rs_ctas = int(os.environ.get("LLMC_RS_CTAS", "32"))
        if os.environ.get("LLMC_RS_THREADS") == "128":
            self.rs_ctas = torch.cuda.get_device_properties(dev).multi_processor_count
        # the last reduction of a step (embeddings, final norm) runs after backward, alone on the GPU: it gets a wider grid
        self.rs_tail_ctas = max(self.rs_ctas, int(os.environ.get("LLMC_RS_TAIL_CTAS", "128")))
        # 2: a one-warp kernel exchanges the "gradients final" flags ahead of the wide kernel, which then never holds SMs while
        # the slowest peer is still computing; 1: the wide kernel does it itself (kept selectable for measurements)
        self.rs_wait_mode = 2 if os.environ.get("LLMC_RS_HANDSHAKE", "1") != "0" else 1
        self.rs_partials = self.lib.llmc_p2p_rs_partials(self.rs_tail_ctas)     # per-channel stride; unused entries stay zero
        self.rs_mode = os.environ.get("LLMC_RS_MODE", "deferred")               # "deferred" | "instream" | "side"
        if self.rs_mode not in ("deferred", "instream", "side"):
            raise ValueError("LLMC_RS_MODE must be deferred, instream or side")
        self._pending = None
        self.num_channels = model.cfg.num_layers + 1
        self.norm_partials = torch.zeros(self.num_channels * self.rs_partials, dtype=torch.float32, device=dev)
        self.done_counter = torch.zeros(2, dtype=torch.int32, device=dev)      # [0] update + gather, [1] all-reduce (other stream)
        self.host_scalar = torch.zeros(1, dtype=torch.float32, device=dev)
        self.seq = 0            # optimizer-step sequence number shared by all flags of a step
        self.scalar_seq = 0
        self.barrier_seq = 0
        self.reduced_this_step = False
        self.published_seq = 0  # sequence number of the last parameter publication (0: parameters are local, nothing to wait for)
        model.param_sync = ParamSync(self)
        torch.cuda.synchronize()
        dist.barrier()          # every rank's buffers are zeroed and mapped before any kernel touches a peer

    # ---- ZeRO-1 backend interface (see zero.py)
    def reduce_tensors(self, grads_flat, slices, channel=None, tail=False):
        if not self.reduced_this_step:
            self.seq += 1
            self.reduced_this_step = True
        ch = self._channel_of(slices)
        self._channels_this_step = max(getattr(self, "_channels_this_step", 0), ch + 1)
        cur = torch.cuda.current_stream()
        mode = self.rs_mode
        if mode == "side":
            # the whole reduction runs on the communication stream, beside the rest of backward
            self.stream.wait_stream(cur)
            if self.rs_wait_mode == 2:
                self._handshake(ch, self.stream)
            self._launch_reduce(slices, ch, self.rs_tail_ctas if tail else self.rs_ctas, self.rs_wait_mode, self.stream)
            return
        # "deferred": only the flag exchange runs on the communication stream (one warp, no SM held); the wide reduction of a
        # layer is launched on the compute stream one layer later, when the exchange has normally long finished, so that it
        # runs alone on the whole GPU for a few tens of microseconds instead of beside a persistent GEMM
        self.stream.wait_stream(cur)
        self._handshake(ch, self.stream)
        ev = torch.cuda.Event()
        ev.record(self.stream)
        self._flush_pending(cur)
        self._pending = (slices, ch, ev)
        if tail or mode == "instream":
            self._flush_pending(cur)

    def _handshake(self, ch, stream):
        kernels._launches += 1
        check(self.lib.llmc_p2p_rs_handshake(self.c_sig, self.r, self.N, ch, self.seq, ctypes.c_void_p(stream.cuda_stream)),
              "llmc_p2p_rs_handshake")

    def _flush_pending(self, cur):
        if self._pending is None:
            return
        slices, ch, ev = self._pending
        self._pending = None
        cur.wait_event(ev)
        self._launch_reduce(slices, ch, self.rs_tail_ctas, 2, cur)

    def _launch_reduce(self, slices, ch, ctas, wait_mode, stream):
        offs = (ctypes.c_longlong * len(slices))(*[s[0] for s in slices])
        sizes = (ctypes.c_longlong * len(slices))(*[s[1] for s in slices])
        kernels._launches += 1
        part = self.norm_partials[ch * self.rs_partials:(ch + 1) * self.rs_partials]
        check(self.lib.llmc_p2p_reduce_scatter(self.c_grads, self.c_sig, offs, sizes, len(slices), self.r, self.N, ch, self.seq,
                                               ctypes.c_void_p(part.data_ptr()), ctas, wait_mode, int(self.zero_stage == 0),
                                               ctypes.c_void_p(self.done_counter.data_ptr() + 4),
                                               ctypes.c_void_p(stream.cuda_stream)), "llmc_p2p_reduce_scatter")

    def _channel_of(self, slices):
        key = slices[0][0]
        if not hasattr(self, "_chan_map"):
            self._chan_map = {}
        if key not in self._chan_map:
            self._chan_map[key] = len(self._chan_map)
            assert self._chan_map[key] < self.num_channels
        return self._chan_map[key]

    def finish_reduce(self):
        cur = torch.cuda.current_stream()
        self._flush_pending(cur)
        cur.wait_stream(self.stream)
        if self.zero_stage == 0 and self.reduced_this_step:
            # data parallel without sharding: every peer's shard of the mean must have landed in this rank's buffer
            kernels._launches += 1
            check(self.lib.llmc_p2p_wait_range(self.c_sig, self.r, self.N, 2, 0, self._channels_this_step, self.seq,
                                               ctypes.c_void_p(cur.cuda_stream)), "llmc_p2p_wait_range")

    def fused_norm_sq(self, scalars, losses=None, loss_scale=1.0):
        """scalars[0] = sum over ranks of the sum of squares of the reduced shards (partials written by the reduce kernels);
        with ``losses``, scalars[1] = sum over ranks of loss_scale * sum(losses).  One launch, one exchange."""
        self.scalar_seq += 1
        kernels._launches += 1
        count = 2 if (losses is not None or scalars.numel() >= 2) else 1
        check(self.lib.llmc_p2p_allreduce_scalars(self.c_sig, kernels._p(scalars), count, kernels._p(self.norm_partials),
                                                  self.norm_partials.numel(), kernels._p(losses), losses.numel() if losses is not None else 0,
                                                  float(loss_scale), self.r, self.N, self.scalar_seq,
                                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "llmc_p2p_allreduce_scalars")

    def all_reduce_scalar_sum(self, t):
        """Sum over ranks, in place, of the first min(t.numel(), 4) floats of a device tensor."""
        self.scalar_seq += 1
        kernels._launches += 1
        check(self.lib.llmc_p2p_allreduce_scalars(self.c_sig, kernels._p(t), min(t.numel(), 4), None, 0, None, 0, 1.0, self.r, self.N,
                                                  self.scalar_seq, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
              "llmc_p2p_allreduce_scalars")
        return t

    def host_float_sum(self, value):
        """Sum of a host float over all ranks (validation loss, evaluation counts; reference: multi_gpu_cpu_float_sum)."""
        self.host_scalar.fill_(float(value))
        self.all_reduce_scalar_sum(self.host_scalar)
        return float(self.host_scalar.item())

    def end_step(self, updated):
        """Closes the bookkeeping of one optimizer step, whether or not the update ran.  The next step's reductions get a new
        sequence number; after a skipped update a device-side barrier keeps every rank from overwriting gradients that a
        slower peer's reduction kernels may still be reading."""
        if self.reduced_this_step and not updated:
            self.barrier()
        self.reduced_this_step = False
        self._channels_this_step = 0

    # ---- parameter groups of the fused update + all-gather, in the order the forward pass consumes them:
    #      group 0 = everything the forward pass touches before / outside the layer GEMMs (embeddings, final norm, LM head and the
    #      small per-layer norm parameters), group 1 + l = the matrices and biases of layer l.
    def _groups(self, views):
        L = self.model.cfg.num_layers
        early = getattr(self.model, "norm_params", ())
        shared, layers = [], [[] for _ in range(L)]
        for v in views:
            if v["L"] == 1 or v["name"] in early:
                shared.append(v)
            else:
                for l in range(v["L"]):
                    w = dict(v)
                    w.update(p_base=v["p_base"] + l * v["p_stride"], o_base=v["o_base"] + l * v["o_stride"], L=1, l_base=l)
                    layers[l].append(w)
        return [shared] + layers

    def adamw_allgather(self, master, m, v, views, lr, beta1, beta2, eps, t, grad_scale, norm_sq, grad_clip):
        """AdamW on the own shards and peer stores of the rounded parameters, one launch per parameter group; each launch raises
        the group's flags on every peer when its stores are out.  Nothing waits here: the consumers do (``ParamSync``)."""
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for ch, group in enumerate(self._groups(views)):
            if not group:
                continue
            tab = kernels.make_table(group)
            kernels._launches += 1
            check(self.lib.llmc_p2p_adamw_allgather(self.c_params, self.c_sig, kernels._p(master), kernels._p(self.grads_t), kernels._p(m),
                                                    kernels._p(v), ctypes.byref(tab), self.r, self.N, lr, beta1, beta2, eps, int(t), grad_scale,
                                                    kernels._p(norm_sq), grad_clip, self.seq, kernels._p(self.done_counter), 4 * self.ctas, ch,
                                                    st), "llmc_p2p_adamw_allgather")
        self.published_seq = self.seq

    def wait_params(self, channel=None):
        """Tiny wait kernel on the current stream: all groups, or one (0 = shared group, 1 + l = layer l)."""
        if self.published_seq == 0:
            return
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        kernels._launches += 1
        if channel is None:
            check(self.lib.llmc_p2p_wait_range(self.c_sig, self.r, self.N, 0, 0, self.model.cfg.num_layers + 1, self.published_seq, st),
                  "llmc_p2p_wait_range")
        else:
            check(self.lib.llmc_p2p_wait(self.c_sig, self.r, self.N, 0, channel, self.published_seq, st), "llmc_p2p_wait")

    def flag_address(self, channel):
        return self.sig_ptrs[self.r] + 8 * self.lib.llmc_p2p_ag_flag_offset(channel)

    def all_gather_slices(self, params_flat, slices):
        raise RuntimeError("the P2P backend gathers inside adamw_allgather")

    def barrier(self):
        """Device-side barrier on the current stream (reference: multi_gpu_barrier)."""
        self.barrier_seq += 1
        kernels._launches += 2
        check(self.lib.llmc_p2p_barrier(self.c_sig, self.r, self.N, self.barrier_seq,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "llmc_p2p_barrier")

    def host_barrier(self):
        """Barrier that the host also waits for (before a checkpoint's DONE marker is written)."""
        self.barrier()
        torch.cuda.current_stream().synchronize()


def try_create(model_factory_args, dist_cfg, zero_stage, log=print):
    """Returns (arena, flat buffers) prerequisites for the P2P backend or None if symmetric memory is unavailable or the
    configuration is not data parallelism (with or without ZeRO-1) on <= 8 ranks of one node."""
    if zero_stage not in (0, 1) or dist_cfg.num_processes > MAX_RANKS or dist_cfg.device.type != "cuda":
        return None
    try:
        return SymmetricArena(dist_cfg)
    except Exception as e:  # pragma: no cover - depends on driver / fabric support
        log("symmetric memory unavailable (%s): falling back to the NCCL backend" % e)
        return None
