"""Parses ``main.log`` into its streams (reference: dev/vislog.ipynb): ``trl`` train loss, ``tel`` validation loss,
``eval`` HellaSwag accuracy, ``lr``, ``norm``; and checks a run's losses against expected values
(reference: dev/loss_checker_ci.py)."""
import re


def parse_logfile(path):
    streams = {}
    with open(path) as f:
        for line in f:
            parts = line.split()
            if not parts or not parts[0].startswith("s:"):
                continue
            step = int(parts[0][2:])
            for kv in parts[1:]:
                k, v = kv.split(":")
                streams.setdefault(k, {})[step] = float(v)
    return streams


STEP_LINE = re.compile(r"step\s+(\d+)/(\d+) \| loss ([0-9.]+) ")


def losses_from_stdout(text):
    """Loss per step from the trainer's stdout (the ``step N/M | loss ...`` lines)."""
    return [float(m.group(3)) for m in STEP_LINE.finditer(text)]


def check_losses(losses, expected, rel_tol=0.05):
    """True if every loss is within rel_tol of the expected one."""
    if len(losses) < len(expected):
        return False
    return all(abs(a - b) <= rel_tol * abs(b) for a, b in zip(losses, expected))
