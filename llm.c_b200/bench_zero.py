"""ZeRO-1 optimizer-step micro-benchmark on a flat buffer the size of GPT-2 1558M (about 1.56 B parameters):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P -m llmc_b200.bench_zero

Inputs per rank: bf16 gradients ~ N(0, 1e-3), fp32 master weights ~ N(0, 0.02), fp32 Adam m / v shards.
Measured, device-timed (CUDA events), max over ranks:
  p2p   this library's kernels: reduce-scatter (peer loads, 1/N scale, norm^2 partials) -> one-shot scalar all-reduce ->
        AdamW + stochastic rounding + all-gather (peer stores)
  nccl  ncclReduceScatter(avg) -> norm^2 kernel + ncclAllReduce -> AdamW kernel -> ncclAllGather   (the reference's scheme)
and reported against the NVLink roofline: (N-1)/N of the bf16 buffer must enter each GPU during the reduce-scatter and
leave it during the all-gather; at 770 GB/s per direction (measured peer-copy rate on this pool) that is the floor.
"""
import ctypes
import json
import sys

import torch
import torch.distributed as dist

from . import _lib
from .ops import kernels
from .parallel import dist as pdist
from .parallel import p2p

NUM_PARAMS = 1_557_594_112          # multiple of 16 * 8 * 8, about GPT-2 1558M
LINK_GBS = 770.0


def main():
    d = pdist.init_distributed(device_type="cuda")
    N, r, dev = d.num_processes, d.process_rank, d.device
    if N < 2:
        raise SystemExit("needs at least two ranks")
    lib = p2p._cfg_lib()
    n = NUM_PARAMS
    shard = n // N
    arena = p2p.SymmetricArena(d)
    params, p_ptrs, _ph = arena.alloc(n, torch.bfloat16)
    grads, g_ptrs, _gh = arena.alloc(n, torch.bfloat16)
    sig, s_ptrs, _sh = arena.alloc(lib.llmc_p2p_signal_words(), torch.int64)
    gen = torch.Generator(device=dev).manual_seed(1 + r)
    master = torch.randn(shard, device=dev, generator=gen) * 0.02
    m, v = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    g_src = (torch.randn(n, device=dev, generator=gen) * 1e-3).to(torch.bfloat16)
    c_p, c_g, c_s = p2p._ptr_array(p_ptrs), p2p._ptr_array(g_ptrs), p2p._ptr_array(s_ptrs)
    slices = 16
    per = n // slices
    offs = (ctypes.c_longlong * slices)(*[i * per for i in range(slices)])
    sizes = (ctypes.c_longlong * slices)(*[per] * slices)
    ctas = 4 * torch.cuda.get_device_properties(dev).multi_processor_count
    lib.llmc_p2p_rs_partials.restype = ctypes.c_int
    lib.llmc_p2p_rs_partials.argtypes = [ctypes.c_int]
    partials = torch.zeros(lib.llmc_p2p_rs_partials(ctas), device=dev)      # one partial sum of squares per warp of the reduce-scatter CTAs
    norm_sq = torch.zeros(1, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    # shard views of the 16 slices (ZeRO-1 layout: rank r owns [r*per/N, (r+1)*per/N) of every slice)
    sh = per // N
    views = [dict(p_base=i * per + r * sh, p_stride=per, o_base=i * sh, o_stride=sh, n=sh, L=1, wd=0.1, seed=17 + i) for i in range(slices)]
    tab = kernels.make_table(views)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    seq = [0, 0]

    def step_p2p():
        seq[0] += 1
        _lib.check(lib.llmc_p2p_reduce_scatter(c_g, c_s, offs, sizes, slices, r, N, 0, seq[0], ctypes.c_void_p(partials.data_ptr()), ctas, 1, 0, None,
                                               stream), "rs")
        seq[1] += 1
        # one launch: sum of the partial sums of squares, then the exchange over the ranks
        _lib.check(lib.llmc_p2p_allreduce_scalars(c_s, ctypes.c_void_p(norm_sq.data_ptr()), 1, ctypes.c_void_p(partials.data_ptr()), partials.numel(),
                                                  None, 0, 1.0, r, N, seq[1], stream), "ar")
        _lib.check(lib.llmc_p2p_adamw_allgather(c_p, c_s, kernels._p(master), kernels._p(grads), kernels._p(m), kernels._p(v), ctypes.byref(tab), r, N,
                                                6e-4, 0.9, 0.95, 1e-8, 1, 1.0, kernels._p(norm_sq), 1.0, seq[0], kernels._p(counter), ctas, 0, stream), "adamw_ag")
        _lib.check(lib.llmc_p2p_wait(c_s, r, N, 0, 0, seq[0], stream), "wait")

    def step_nccl():
        for i in range(slices):
            full = grads[i * per:(i + 1) * per]
            dist.reduce_scatter_tensor(full[r * sh:(r + 1) * sh], full, op=dist.ReduceOp.AVG)
        kernels.global_norm_sq(norm_sq, grads, views)
        dist.all_reduce(norm_sq)
        kernels.adamw_update(params, master, grads, m, v, views, 6e-4, 0.9, 0.95, 1e-8, 1, 1.0, norm_sq, 1.0)
        for i in range(slices):
            full = params[i * per:(i + 1) * per]
            dist.all_gather_into_tensor(full, full[r * sh:(r + 1) * sh].clone())

    def timed(fn, iters=5, warm=2):
        ts = []
        for it in range(warm + iters):
            grads.copy_(g_src)
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            if it >= warm:
                ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_p2p = timed(step_p2p)
    t_nccl = timed(step_nccl)
    status = _lib.read_status()
    link_bytes = 2.0 * n * (N - 1) / N                      # per direction, per phase (reduce-scatter in, all-gather out)
    floor_ms = 2 * link_bytes / (LINK_GBS * 1e9) * 1e3      # the two phases cannot overlap: the norm sits between them
    if r == 0:
        print(json.dumps({"bench": "zero1_step_1558M_flat", "n_gpus": N, "params": n, "p2p_ms": t_p2p, "nccl_ms": t_nccl, "speedup_vs_nccl": t_nccl / t_p2p,
                          "nvlink_floor_ms": floor_ms, "p2p_fraction_of_nvlink_roofline": floor_ms / t_p2p, "kernel_status": status}), flush=True)
    pdist.shutdown(d)


if __name__ == "__main__":
    sys.exit(main())
