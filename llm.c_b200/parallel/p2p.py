"""ZeRO-1 communication backend that runs this library's own kernels over NVLink peer memory (csrc/comm.cu).

The flat parameter and gradient buffers and one small signal buffer are allocated as symmetric memory
(``torch.distributed._symmetric_memory``: same size on every rank, every rank can address every peer's copy).
NCCL is used only to rendezvous and to exchange the buffer handles.  After that a training step issues no NCCL
call: the per-layer gradient reduce-scatter (fused with the 1/N scale and the norm^2 partial sums), the scalar
all-reduce of the norm and the AdamW update fused with the all-gather of the rounded bf16 parameters are all
kernels that load from / store to peer memory directly.

Capability parity: multi_gpu_async_reduce_gradient, the ncclAllReduce of the norm and the ncclAllGather of
gpt2_update in the reference (llmc/zero.cuh:528-551, train_gpt2.cu:1002-1030 and 1101-1120).
"""
import ctypes

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
        lib.llmc_p2p_reduce_scatter.argtypes = [P, P, P, P, I, I, I, I, U, P, I, I, P]
        lib.llmc_p2p_allreduce_scalar.restype = I
        lib.llmc_p2p_allreduce_scalar.argtypes = [P, P, I, I, U, P]
        lib.llmc_p2p_adamw_allgather.restype = I
        lib.llmc_p2p_adamw_allgather.argtypes = [P, P, P, P, P, P, ctypes.POINTER(_lib.TensorTable), I, I, F, F, F, F, I, F, P, F, U, P, I, P]
        lib.llmc_p2p_wait.restype = I
        lib.llmc_p2p_wait.argtypes = [P, I, I, I, U, P]
        lib.llmc_p2p_barrier.restype = I
        lib.llmc_p2p_barrier.argtypes = [P, I, I, U, P]
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


class P2PBackend:
    name = "p2p"

    def __init__(self, model, dist_cfg, arena, params, grads):
        self.cfg = dist_cfg
        self.N, self.r = dist_cfg.num_processes, dist_cfg.process_rank
        self.lib = _cfg_lib()
        self.model = model
        self.params_t, self.param_ptrs, self._ph = params
        self.grads_t, self.grad_ptrs, self._gh = grads
        words = self.lib.llmc_p2p_signal_words()
        self.sig_t, self.sig_ptrs, self._sh = arena.alloc(words, torch.int64)
        self.c_params, self.c_grads, self.c_sig = _ptr_array(self.param_ptrs), _ptr_array(self.grad_ptrs), _ptr_array(self.sig_ptrs)
        dev = dist_cfg.device
        self.stream = torch.cuda.Stream(device=dev)
        self.ctas = 32
        self.num_channels = model.cfg.num_layers + 1
        self.norm_partials = torch.zeros(self.num_channels * self.ctas, dtype=torch.float32, device=dev)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.seq = 0            # optimizer-step sequence number shared by all flags of a step
        self.scalar_seq = 0
        self.barrier_seq = 0
        self.reduced_this_step = False
        torch.cuda.synchronize()
        dist.barrier()          # every rank's buffers are zeroed and mapped before any kernel touches a peer

    # ---- ZeRO-1 backend interface (see zero.py)
    def reduce_tensors(self, grads_flat, slices, channel=None):
        if not self.reduced_this_step:
            self.seq += 1
            self.reduced_this_step = True
        ch = self._channel_of(slices)
        offs = (ctypes.c_longlong * len(slices))(*[s[0] for s in slices])
        sizes = (ctypes.c_longlong * len(slices))(*[s[1] for s in slices])
        self.stream.wait_stream(torch.cuda.current_stream())
        kernels._launches += 1
        part = self.norm_partials[ch * self.ctas:(ch + 1) * self.ctas]
        check(self.lib.llmc_p2p_reduce_scatter(self.c_grads, self.c_sig, offs, sizes, len(slices), self.r, self.N, ch, self.seq,
                                               ctypes.c_void_p(part.data_ptr()), self.ctas, 1,
                                               ctypes.c_void_p(self.stream.cuda_stream)), "llmc_p2p_reduce_scatter")

    def _channel_of(self, slices):
        key = slices[0][0]
        if not hasattr(self, "_chan_map"):
            self._chan_map = {}
        if key not in self._chan_map:
            self._chan_map[key] = len(self._chan_map)
            assert self._chan_map[key] < self.num_channels
        return self._chan_map[key]

    def finish_reduce(self):
        torch.cuda.current_stream().wait_stream(self.stream)

    def fused_norm_sq(self, out):
        """out[0] = sum over ranks of the sum of squares of the reduced shards (partials written by the reduce kernels)."""
        torch.sum(self.norm_partials, dim=0, keepdim=True, out=out)
        self.all_reduce_scalar_sum(out)

    def all_reduce_scalar_sum(self, t):
        self.scalar_seq += 1
        kernels._launches += 1
        check(self.lib.llmc_p2p_allreduce_scalar(self.c_sig, ctypes.c_void_p(t.data_ptr()), self.r, self.N, self.scalar_seq,
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "llmc_p2p_allreduce_scalar")
        return t

    def adamw_allgather(self, master, m, v, views, lr, beta1, beta2, eps, t, grad_scale, norm_sq, grad_clip):
        tab = kernels.make_table(views)
        kernels._launches += 2
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(self.lib.llmc_p2p_adamw_allgather(self.c_params, self.c_sig, kernels._p(master), kernels._p(self.grads_t), kernels._p(m),
                                                kernels._p(v), ctypes.byref(tab), self.r, self.N, lr, beta1, beta2, eps, int(t), grad_scale,
                                                kernels._p(norm_sq), grad_clip, self.seq, kernels._p(self.done_counter), 4 * self.ctas, st),
              "llmc_p2p_adamw_allgather")
        # the next consumer of the parameters (the following forward) runs after every peer has published its shards
        check(self.lib.llmc_p2p_wait(self.c_sig, self.r, self.N, 0, self.seq, st), "llmc_p2p_wait")
        self.reduced_this_step = False

    def all_gather_slices(self, params_flat, slices):
        raise RuntimeError("the P2P backend gathers inside adamw_allgather")

    def barrier(self):
        self.barrier_seq += 1
        check(self.lib.llmc_p2p_barrier(self.c_sig, self.r, self.N, self.barrier_seq,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "llmc_p2p_barrier")


def try_create(model_factory_args, dist_cfg, zero_stage, log=print):
    """Returns (arena, flat buffers) prerequisites for the P2P backend or None if symmetric memory is unavailable or the
    configuration is not ZeRO-1 on <= 8 ranks of one node."""
    if zero_stage != 1 or dist_cfg.num_processes > MAX_RANKS or dist_cfg.device.type != "cuda":
        return None
    try:
        return SymmetricArena(dist_cfg)
    except Exception as e:  # pragma: no cover - depends on driver / fabric support
        log("symmetric memory unavailable (%s): falling back to the NCCL backend" % e)
        return None
