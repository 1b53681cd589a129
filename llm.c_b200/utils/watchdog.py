"""Host-side failure detection for long runs.

The reference has none in-process: every error path calls exit() and recovery is the restart loop of its run scripts
(scripts/run_gpt2_124M.sh:12-42 of the reference: re-launch with -y 1 until DONE_<last step> exists).  That loop only helps if
a broken job actually ends.  In synchronous data parallelism one dead or stuck rank leaves all the others blocked in their next
collective, so this module makes "no progress" an error of its own:

  * every rank calls ``beat(step)`` once per optimizer step; the call records the time and atomically rewrites
    ``<log dir>/heartbeat_<rank>.json``;
  * a daemon thread per rank checks the age of the rank's own last beat; past ``timeout_s`` it builds a report (own step, and
    the step and heartbeat age of every peer it can see in the log directory, stalest first) and calls ``on_stall`` -- by
    default it prints the report and ends the process with exit code 17, which the restart loop treats like any other failure.

Device-side waits are bounded separately (kernels give up and set a status word); the trainer turns a non-zero status word into
an exception at the end of the step.  Nothing here touches a GPU.
"""
import json
import os
import sys
import threading
import time

EXIT_STALLED = 17


class StepWatchdog:
    def __init__(self, log_dir, rank, world, timeout_s, on_stall=None, poll_s=None):
        self.log_dir, self.rank, self.world, self.timeout_s = log_dir, rank, world, float(timeout_s)
        self.on_stall = on_stall or self._default_on_stall
        self.poll_s = poll_s if poll_s is not None else max(0.05, min(1.0, self.timeout_s / 4.0))
        self.last_beat = time.time()
        self.step, self.phase = -1, "start"
        self._stop = threading.Event()
        self._thread = None
        self.fired = False
        if log_dir:
            os.makedirs(log_dir, exist_ok=True)

    def path(self, rank=None):
        return os.path.join(self.log_dir, "heartbeat_%05d.json" % (self.rank if rank is None else rank))

    # ---- called by the training loop
    def beat(self, step, phase="step"):
        self.last_beat, self.step, self.phase = time.time(), int(step), phase
        if self.log_dir:
            tmp = self.path() + ".tmp"
            with open(tmp, "w") as f:
                json.dump({"rank": self.rank, "step": self.step, "phase": phase, "time": self.last_beat, "pid": os.getpid()}, f)
            os.replace(tmp, self.path())

    def start(self):
        if self.timeout_s > 0 and self._thread is None:
            self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
            self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None

    # ---- the monitor
    def peers(self):
        """[(rank, step, age in seconds)] of every rank with a readable heartbeat file, stalest first."""
        now, out = time.time(), []
        if not self.log_dir:
            return out
        for r in range(self.world):
            try:
                with open(self.path(r)) as f:
                    hb = json.load(f)
                out.append((r, int(hb["step"]), now - float(hb["time"])))
            except (OSError, ValueError, KeyError):
                out.append((r, None, float("inf")))
        return sorted(out, key=lambda x: -x[2])

    def report(self):
        age = time.time() - self.last_beat
        lines = ["[watchdog] rank %d: no progress for %.1f s (limit %.1f s); last completed step %d, phase %s"
                 % (self.rank, age, self.timeout_s, self.step, self.phase)]
        for r, step, a in self.peers():
            lines.append("[watchdog]   rank %d: %s" % (r, "no heartbeat file" if step is None else "step %d, heartbeat %.1f s old" % (step, a)))
        return "\n".join(lines)

    def _run(self):
        while not self._stop.wait(self.poll_s):
            if time.time() - self.last_beat > self.timeout_s:
                self.fired = True
                self.on_stall(self.report())
                return

    @staticmethod
    def _default_on_stall(report):
        print(report, file=sys.stderr, flush=True)
        os._exit(EXIT_STALLED)
