"""Data parallelism on real GPUs: the in-kernel NVLink path (P2P reduce-scatter or all-reduce / fused AdamW + all-gather /
one-shot scalar all-reduce) against the NCCL path and against a single-GPU run with gradient accumulation, on 2, 4 and 8
GPUs (each case is skipped where the machine has fewer)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "dist_worker.py")


def launch(world, out, extra, port, timeout=600, env_extra=None):
    env = dict(os.environ)
    env.update(env_extra or {})
    if world == 1:
        cmd = [sys.executable, WORKER, "--out", out] + extra
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
               "--master-port", str(port), WORKER, "--out", out] + extra
    return subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)


def need(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_p2p_and_nccl_zero1_match_single_gpu(tmp_path, world):
    need(world)
    single, nccl, p2p = (str(tmp_path / n) for n in ("single.pt", "nccl.pt", "p2p.pt"))
    r = launch(1, single, ["--device", "cuda", "--zero", "0", "--slots", str(world)], 0)
    assert r.returncode == 0, r.stdout[-3000:]
    r = launch(world, nccl, ["--device", "cuda", "--zero", "1", "--slots", str(world), "--backend", "nccl"], 29541)
    assert r.returncode == 0, r.stdout[-3000:]
    r = launch(world, p2p, ["--device", "cuda", "--zero", "1", "--slots", str(world), "--backend", "p2p"], 29542)
    assert r.returncode == 0, r.stdout[-3000:]
    # the same run with every GEMM on the two-SM kernel: the first GEMM of each layer then polls the all-gather flags inside the kernel
    p2p_fused = str(tmp_path / "p2p_fused.pt")
    r = launch(world, p2p_fused, ["--device", "cuda", "--zero", "1", "--slots", str(world), "--backend", "p2p"], 29543,
               env_extra={"LLMC_GEMM_2SM_MIN_TILES": "1"})
    assert r.returncode == 0, r.stdout[-3000:]
    pf = torch.load(p2p_fused)
    s, n, p = torch.load(single), torch.load(nccl), torch.load(p2p)
    assert pf["backend"] == "p2p"
    assert max(abs(x - y) for x, y in zip(p["losses"], pf["losses"])) < 2e-2
    assert (p["params"] - pf["params"]).abs().max().item() < 2e-2
    assert p["backend"] == "p2p" and n["backend"] == "nccl" and p["zero"] == 1
    for other in (n, p):
        assert max(abs(x - y) for x, y in zip(s["losses"], other["losses"])) < 3e-2, (s["losses"], other["losses"])
        diff = (s["params"] - other["params"]).abs().max().item()
        assert diff < 2e-2, diff
    # the two communication paths compute the same mean of the same bf16 gradients
    assert max(abs(x - y) for x, y in zip(n["losses"], p["losses"])) < 2e-2
    assert s["losses"][-1] < s["losses"][0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_llama_p2p_zero1_matches_single_gpu(tmp_path):
    """The LLaMA-3 family under ZeRO-1 on the in-kernel NVLink path (its parameter groups differ from GPT-2's: no biases, an untied
    head in the shared group) against a single-GPU run with gradient accumulation."""
    world = 2
    single, p2p = str(tmp_path / "single.pt"), str(tmp_path / "p2p.pt")
    r = launch(1, single, ["--device", "cuda", "--zero", "0", "--slots", str(world), "--family", "llama3"], 0)
    assert r.returncode == 0, r.stdout[-3000:]
    r = launch(world, p2p, ["--device", "cuda", "--zero", "1", "--slots", str(world), "--backend", "p2p", "--family", "llama3"], 29551,
               env_extra={"LLMC_GEMM_2SM_MIN_TILES": "1"})
    assert r.returncode == 0, r.stdout[-3000:]
    s, p = torch.load(single), torch.load(p2p)
    assert p["backend"] == "p2p" and p["zero"] == 1
    assert max(abs(x - y) for x, y in zip(s["losses"], p["losses"])) < 3e-2, (s["losses"], p["losses"])
    assert (s["params"] - p["params"]).abs().max().item() < 2e-2


@pytest.mark.parametrize("world", [2, 4])
def test_p2p_allreduce_without_sharding_matches_single_gpu(tmp_path, world):
    """-z 0 on the in-kernel path: the reduction kernel stores the mean into every rank's gradient buffer (all-reduce) and every
    rank updates a full replica."""
    need(world)
    single, p2p = str(tmp_path / "single.pt"), str(tmp_path / "p2p.pt")
    r = launch(1, single, ["--device", "cuda", "--zero", "0", "--slots", str(world)], 0)
    assert r.returncode == 0, r.stdout[-3000:]
    r = launch(world, p2p, ["--device", "cuda", "--zero", "0", "--slots", str(world), "--backend", "p2p"], 29561)
    assert r.returncode == 0, r.stdout[-3000:]
    s, p = torch.load(single), torch.load(p2p)
    assert p["backend"] == "p2p" and p["zero"] == 0
    assert max(abs(x - y) for x, y in zip(s["losses"], p["losses"])) < 3e-2, (s["losses"], p["losses"])
    assert (s["params"] - p["params"]).abs().max().item() < 2e-2


def test_skipped_update_keeps_the_two_backends_in_step(tmp_path):
    """A step whose update is skipped on the host (the outlier detector's decision) must leave the flag sequence numbers of the
    in-kernel path consistent: the following steps still match the NCCL path."""
    world = 2
    need(world)
    nccl, p2p = str(tmp_path / "nccl.pt"), str(tmp_path / "p2p.pt")
    common = ["--device", "cuda", "--zero", "1", "--slots", str(world), "--steps", "5", "--skip-step", "2"]
    r = launch(world, nccl, common + ["--backend", "nccl"], 29571)
    assert r.returncode == 0, r.stdout[-3000:]
    r = launch(world, p2p, common + ["--backend", "p2p"], 29572)
    assert r.returncode == 0, r.stdout[-3000:]
    n, p = torch.load(nccl), torch.load(p2p)
    assert p["backend"] == "p2p"
    assert max(abs(x - y) for x, y in zip(n["losses"], p["losses"])) < 2e-2, (n["losses"], p["losses"])
    assert (n["params"] - p["params"]).abs().max().item() < 2e-2
    assert n["losses"][3] == pytest.approx(n["losses"][2], abs=0.3)      # nothing moved between step 2 and 3 but the batch
