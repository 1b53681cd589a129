"""Parses ``main.log`` into its streams (reference: dev/vislog.ipynb): ``trl`` train loss, ``tel`` validation loss,
``eval`` HellaSwag accuracy, ``lr``, ``norm``; plots them against the published GPT-2 / GPT-3 baselines (the notebook's figure);
and checks a run's losses against expected values (reference: dev/loss_checker_ci.py).

    python -m llmc_b200.utils.vislog log124M/main.log --model 124M --out curves.png
"""
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


# Baselines the reference's notebook draws as horizontal lines (dev/vislog.ipynb, cell 4): validation loss of the OpenAI
# checkpoints on the FineWeb validation split, and HellaSwag accuracies of GPT-2 / GPT-3 models of the same size.
LOSS_BASELINE = {"124M": 3.4250, "350M": 3.0831, "774M": 3.0006, "1558M": 2.8313}
HELLA2_BASELINE = {"124M": 0.2945, "350M": 0.3752, "774M": 0.4320, "1558M": 0.4889}
HELLA3_BASELINE = {"124M": 0.337, "350M": 0.436, "774M": 0.510, "1558M": 0.547}


def plot_log(path, model="124M", out_path=None, ylim_loss=None):
    """Two panels like the notebook: train / validation loss with the OpenAI checkpoint's validation loss as a line, and
    HellaSwag accuracy with the GPT-2 and GPT-3 lines.  Returns the matplotlib figure (needs matplotlib; the parser above does not)."""
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    st = parse_logfile(path)
    fig, axes = plt.subplots(1, 2, figsize=(16, 6))
    ax = axes[0]
    if "trl" in st:
        xs, ys = zip(*sorted(st["trl"].items()))
        ax.plot(xs, ys, label="llm.c_b200 (%s) train loss" % model, alpha=0.6)
    if "tel" in st:
        xs, ys = zip(*sorted(st["tel"].items()))
        ax.plot(xs, ys, label="llm.c_b200 (%s) val loss" % model)
    if model in LOSS_BASELINE:
        ax.axhline(LOSS_BASELINE[model], color="r", linestyle="--", label="OpenAI GPT-2 (%s) checkpoint val loss" % model)
    ax.set_xlabel("steps"); ax.set_ylabel("loss"); ax.set_yscale("log"); ax.set_title("Loss"); ax.legend()
    if ylim_loss:
        ax.set_ylim(*ylim_loss)
    ax = axes[1]
    if "eval" in st:
        xs, ys = zip(*sorted(st["eval"].items()))
        ax.plot(xs, ys, label="llm.c_b200 (%s)" % model)
    if model in HELLA2_BASELINE:
        ax.axhline(HELLA2_BASELINE[model], color="r", linestyle="--", label="OpenAI GPT-2 (%s) checkpoint" % model)
        ax.axhline(HELLA3_BASELINE[model], color="g", linestyle="--", label="OpenAI GPT-3 (%s) checkpoint" % model)
    ax.set_xlabel("steps"); ax.set_ylabel("accuracy"); ax.set_title("HellaSwag eval"); ax.legend()
    if out_path:
        fig.savefig(out_path, dpi=100, bbox_inches="tight")
    return fig


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="plot the streams of a main.log")
    ap.add_argument("log")
    ap.add_argument("--model", default="124M", choices=sorted(LOSS_BASELINE))
    ap.add_argument("--out", default="curves.png")
    a = ap.parse_args(argv)
    st = parse_logfile(a.log)
    for k, v in st.items():
        last = max(v)
        print("%-5s %6d points, last s:%d = %g" % (k, len(v), last, v[last]))
    try:
        plot_log(a.log, a.model, a.out)
        print("wrote %s" % a.out)
    except ImportError:
        print("matplotlib is not installed: no figure written")
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
