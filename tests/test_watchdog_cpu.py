"""Host-side failure detection: heartbeat files, the stall report, and a stalled rank inside a two-rank gloo job ending the
job instead of hanging it.  No GPU is involved."""
import json
import os
import subprocess
import sys
import time

from llmc_b200.utils.watchdog import EXIT_STALLED, StepWatchdog

HERE = os.path.dirname(os.path.abspath(__file__))


def test_heartbeat_file_and_stall_report(tmp_path):
    reports = []
    w0 = StepWatchdog(str(tmp_path), 0, 3, timeout_s=0.3, on_stall=reports.append)
    w1 = StepWatchdog(str(tmp_path), 1, 3, timeout_s=0.0)
    w1.beat(7)
    w0.beat(9, "step")
    with open(w0.path()) as f:
        hb = json.load(f)
    assert hb["rank"] == 0 and hb["step"] == 9 and hb["pid"] == os.getpid()
    w0.start()
    for _ in range(3):                       # progress: no report
        time.sleep(0.1)
        w0.beat(10)
    assert not reports
    time.sleep(0.8)                          # no progress: exactly one report, naming every rank
    w0.stop()
    assert len(reports) == 1 and w0.fired
    rep = reports[0]
    assert "rank 0: no progress" in rep and "last completed step 10" in rep
    assert "rank 1: step 7" in rep and "rank 2: no heartbeat file" in rep
    assert rep.index("rank 2: no heartbeat") < rep.index("rank 1: step 7")       # stalest first


def test_watchdog_off_never_fires(tmp_path):
    reports = []
    w = StepWatchdog(str(tmp_path), 0, 1, timeout_s=0.0, on_stall=reports.append).start()
    time.sleep(0.3)
    w.stop()
    assert not reports and not w.fired


WORKER = r"""
import os, sys, time
sys.path.insert(0, %(root)r)
import torch, torch.distributed as dist
from llmc_b200.utils.watchdog import StepWatchdog
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%(port)d", rank=int(os.environ["RANK"]), world_size=2)
rank = dist.get_rank()
wd = StepWatchdog(%(dir)r, rank, 2, timeout_s=3.0).start()
for step in range(100):
    if rank == 1 and step == 3:
        time.sleep(600)                      # a rank that stops making progress (host-side injection)
    t = torch.ones(1)
    dist.all_reduce(t)                       # rank 0 blocks here once rank 1 is stuck
    wd.beat(step + 1)
print("finished", rank)
"""


def test_stalled_rank_ends_both_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": os.path.dirname(HERE), "port": 29571, "dir": str(tmp_path)})
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(os.environ, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    t0 = time.time()
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    assert time.time() - t0 < 90
    assert [p.returncode for p in procs] == [EXIT_STALLED, EXIT_STALLED], outs
    assert "rank 0: no progress" in outs[0] and "last completed step 3" in outs[0]
    assert "finished" not in outs[0] + outs[1]
