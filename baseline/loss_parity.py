"""This framework and the unmodified reference trainer on the same inputs, side by side.

    python baseline/loss_parity.py --steps 20            # loss curves; one GPU, GPT-2 124M, B=64 T=1024, 524288 tokens per step
    python baseline/loss_parity.py --cross-load          # checkpoints written by one trainer, resumed (-y 1) by the other

Loss curves: both trainers start from the same random initialisation (descriptor d12: the reference's mt19937 draw order is
reproduced bit for bit), read the same synthetic token shards in the same shuffled order (the shard / intra-shard permutations
are the reference's), and use the same hyper-parameters (lr 6e-4, 700 warm-up steps, weight decay 0.1, clip 1.0, bf16 with fp32
master weights).  What differs is every kernel, the stochastic-rounding stream and the summation orders, so the curves agree to
bf16 noise, not bit for bit.  Prints one line per step and the largest difference; exits 0 if that stays below --tol.

Cross-loading: each trainer runs 2*K steps and writes model_*.bin / state_*.bin / DONE_* at step K (reference: train_gpt2.cu
write_checkpoint / load_state); the OTHER trainer is then started with -y 1 on that directory and must continue from step K
with the losses of the run that wrote the files (same tolerance): the model file, the optimizer-state file (m, v, master
weights, random-number state, data-loader position) and the DONE marker are read by a program that did not write them.
"""
import argparse
import os
import re
import subprocess
import sys
import tempfile
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
EXE = os.path.join(ROOT, "baseline", "_ref", "train_gpt2cu")


def losses_from(stdout):
    """{step: loss} from the "step  N/M | loss X" lines both trainers print."""
    return {int(m.group(1)): float(m.group(2)) for m in re.finditer(r"step\s+(\d+)/\d+ \| loss ([0-9.]+)", stdout)}


def common_flags(a, steps, out_dir=None, checkpoint_every=0, resume=0):
    import bench
    geo = types.SimpleNamespace(batch=a.batch, seq=a.seq, total_batch=a.total_batch)
    bench.write_shards(geo)
    train, val = bench.shard_patterns(geo)
    flags = ["-i", train, "-j", val, "-e", a.model, "-b", str(a.batch), "-t", str(a.seq), "-d", str(a.total_batch), "-z", "0",
             "-c", "0.1", "-l", "6e-4", "-u", "700", "-q", "0.0", "-r", "0", "-x", str(steps), "-v", "1000000", "-m", "1",
             "-s", "1000000", "-g", "2", "-h", "0", "-n", str(checkpoint_every), "-y", str(resume)]
    if out_dir:
        flags += ["-o", out_dir]
    return flags


def run_reference(flags):
    sync_dir = tempfile.mkdtemp(prefix="llmc_b200_parity_")
    r = subprocess.run([EXE] + flags + ["-pn", "1", "-pr", "0", "-pg", "8", "-pi", "fs", "-pf", sync_dir], cwd=os.path.dirname(EXE),
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=3000)
    if r.returncode != 0:
        raise RuntimeError("the reference trainer exited with code %d:\n%s" % (r.returncode, r.stdout[-2000:]))
    return losses_from(r.stdout)


def run_ours(flags):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "train_gpt2.py")] + flags, cwd=ROOT, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=3000)
    if r.returncode != 0:
        raise RuntimeError("train_gpt2.py exited with code %d:\n%s" % (r.returncode, r.stdout[-2000:]))
    return losses_from(r.stdout)


def compare(title, want, got, steps, tol, out=sys.stdout):
    """Prints the two curves over `steps`; returns the largest difference (inf when a step is missing)."""
    print(title, file=out)
    worst = 0.0
    for s in steps:
        if s not in want or s not in got:
            print("%4d   missing (%s / %s)" % (s, want.get(s), got.get(s)), file=out)
            worst = float("inf")
            continue
        d = got[s] - want[s]
        worst = max(worst, abs(d))
        print("%4d   %9.6f   %9.6f   %+9.6f" % (s, want[s], got[s], d), file=out)
    print("largest difference: %.6f (tolerance %.3f)" % (worst, tol), file=out, flush=True)
    return worst


def loss_parity(a, out=sys.stdout):
    flags = common_flags(a, a.steps)
    ref, ours = run_reference(flags), run_ours(flags)
    return compare("step   reference        ours        diff", ref, ours, range(1, a.steps + 1), a.tol, out)


def forget_later_checkpoints(directory, K):
    """Both trainers also write a checkpoint at their last step; resuming picks the largest DONE marker, so drop those after K."""
    for name in os.listdir(directory):
        m = re.match(r"DONE_(\d+)$", name)
        if m and int(m.group(1)) > K:
            os.remove(os.path.join(directory, name))


def cross_load(a, out=sys.stdout):
    """Returns the largest loss difference over the resumed halves of both directions."""
    K = a.checkpoint_step
    d_ours, d_ref = tempfile.mkdtemp(prefix="llmc_b200_ckpt_ours_"), tempfile.mkdtemp(prefix="llmc_b200_ckpt_ref_")
    # this framework writes at step K, the reference resumes
    ours_full = run_ours(common_flags(a, 2 * K, d_ours, checkpoint_every=K))
    forget_later_checkpoints(d_ours, K)
    ref_resumed = run_reference(common_flags(a, 2 * K, d_ours, checkpoint_every=0, resume=1))
    if min(ref_resumed) != K + 1:
        raise RuntimeError("the reference did not resume at step %d: its first step line is %d" % (K + 1, min(ref_resumed)))
    w1 = compare("step   ours (writer)   reference (resumed from our files)   diff", ours_full, ref_resumed, range(K + 1, 2 * K + 1), a.tol, out)
    # the reference writes at step K, this framework resumes
    ref_full = run_reference(common_flags(a, 2 * K, d_ref, checkpoint_every=K))
    forget_later_checkpoints(d_ref, K)
    ours_resumed = run_ours(common_flags(a, 2 * K, d_ref, checkpoint_every=0, resume=1))
    if min(ours_resumed) != K + 1:
        raise RuntimeError("train_gpt2.py did not resume at step %d: its first step line is %d" % (K + 1, min(ours_resumed)))
    w2 = compare("step   reference (writer)   ours (resumed from its files)   diff", ref_full, ours_resumed, range(K + 1, 2 * K + 1), a.tol, out)
    return max(w1, w2)


def parse(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--model", default="d12")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--tol", type=float, default=0.02)
    ap.add_argument("--cross-load", action="store_true")
    ap.add_argument("--checkpoint-step", type=int, default=5)
    return ap.parse_args(argv)


def main(argv=None):
    a = parse(argv)
    if not os.path.exists(EXE):
        print("baseline/_ref/train_gpt2cu is not built (see baseline/README.md)")
        return 2
    try:
        worst = cross_load(a) if a.cross_load else loss_parity(a)
    except RuntimeError as e:
        print(e)
        return 2
    return 0 if worst < a.tol else 1


if __name__ == "__main__":
    sys.exit(main())
