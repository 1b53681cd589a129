"""Process bootstrap: one process per GPU, ``torch.distributed`` for the plumbing.

Rank, world size and rendezvous come either from the launcher's environment (torchrun: RANK, WORLD_SIZE,
LOCAL_RANK, MASTER_ADDR, MASTER_PORT) or from the reference's own flags (-pn/-pr/-pg with -pi tcp|fs|mpi,
llmc/zero.cuh:411-466 of the reference): ``tcp`` rendezvous at tcp://<server ip>:12345, ``fs`` through a
file on a shared file system, ``mpi`` through the environment variables an MPI launcher exports.
On CPU (tests) the backend is gloo; on GPUs it is NCCL, which is then used for rendezvous, for handle
exchange of the symmetric buffers and as the measured baseline path.
"""
import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class DistConfig:
    process_rank: int = 0
    num_processes: int = 1
    local_device_idx: int = 0
    device: torch.device = torch.device("cpu")
    initialized_here: bool = False

    @property
    def is_main(self):
        return self.process_rank == 0


def init_distributed(num_processes=1, process_rank=0, gpus_per_node=8, init_method="mpi", server_ip="", fs_path="",
                     device_type=None, timeout_s=600):
    env = os.environ
    if "RANK" in env and "WORLD_SIZE" in env:                          # torchrun
        rank, world = int(env["RANK"]), int(env["WORLD_SIZE"])
        local = int(env.get("LOCAL_RANK", rank % gpus_per_node))
        method = "env://"
    elif init_method == "mpi" and ("OMPI_COMM_WORLD_RANK" in env or "PMI_RANK" in env):
        rank = int(env.get("OMPI_COMM_WORLD_RANK", env.get("PMI_RANK", 0)))
        world = int(env.get("OMPI_COMM_WORLD_SIZE", env.get("PMI_SIZE", 1)))
        local = int(env.get("OMPI_COMM_WORLD_LOCAL_RANK", rank % gpus_per_node))
        method = "tcp://%s:%s" % (env.get("MASTER_ADDR", "127.0.0.1"), env.get("MASTER_PORT", "12345"))
    else:
        rank, world, local = process_rank, num_processes, process_rank % gpus_per_node
        if init_method == "tcp":
            method = "tcp://%s:12345" % (server_ip or "127.0.0.1")
        elif init_method == "fs":
            if not fs_path:
                raise ValueError("-pi fs needs a shared path (-pf)")
            os.makedirs(fs_path, exist_ok=True)
            method = "file://" + os.path.join(os.path.abspath(fs_path), "rendezvous.sync")
        else:
            method = "tcp://127.0.0.1:12345"
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    if device_type == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    cfg = DistConfig(rank, world, local, device, False)
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if device_type == "cuda" else "gloo"
        kwargs = dict(backend=backend, init_method=method, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        if backend == "nccl":
            kwargs["device_id"] = device
        dist.init_process_group(**kwargs)
        cfg.initialized_here = True
    return cfg


def shutdown(cfg):
    if cfg.initialized_here and dist.is_initialized():
        dist.destroy_process_group()


def barrier(cfg):
    if cfg.num_processes > 1:
        dist.barrier()


def host_float_sum(cfg, value):
    """Sum of a host float over all ranks (validation loss, evaluation counts)."""
    if cfg.num_processes == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=cfg.device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
