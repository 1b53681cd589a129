"""Loss curves of this framework and of the unmodified reference trainer on the same inputs, side by side.

    python baseline/loss_parity.py --steps 20            # one GPU, GPT-2 124M, B=64 T=1024, 524288 tokens per step

Both trainers start from the same random initialisation (descriptor d12: the reference's mt19937 draw order is reproduced
bit for bit), read the same synthetic token shards in the same shuffled order (the shard / intra-shard permutations are the
reference's), and use the same hyper-parameters (lr 6e-4, 700 warm-up steps, weight decay 0.1, clip 1.0, bf16 with fp32 master
weights).  What differs is every kernel, the stochastic-rounding stream and the summation orders, so the curves agree to bf16
noise, not bit for bit.  Prints one line per step and the largest difference; exits 0 if that stays below --tol.
"""
import argparse
import os
import re
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def losses_from(stdout):
    return [float(m.group(1)) for m in re.finditer(r"step\s+\d+/\d+ \| loss ([0-9.]+)", stdout)]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--model", default="d12")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--tol", type=float, default=0.02)
    a = ap.parse_args()
    import bench
    exe = os.path.join(ROOT, "baseline", "_ref", "train_gpt2cu")
    if not os.path.exists(exe):
        print("baseline/_ref/train_gpt2cu is not built (see baseline/README.md)")
        return 2
    data_dir = os.path.join(tempfile.gettempdir(), "llmc_b200_bench_data")
    bench.write_shards(data_dir, max(2 * a.total_batch + 1, 4 * 1024 * 1024), a.batch * a.seq * 2 + 1, 1234)
    flags = ["-i", os.path.join(data_dir, "synth_train_*.bin"), "-j", os.path.join(data_dir, "synth_val_*.bin"), "-e", a.model,
             "-b", str(a.batch), "-t", str(a.seq), "-d", str(a.total_batch), "-z", "0", "-c", "0.1", "-l", "6e-4", "-u", "700", "-q", "0.0",
             "-r", "0", "-x", str(a.steps), "-v", "1000000", "-m", "1", "-s", "1000000", "-g", "2", "-h", "0", "-n", "0"]
    sync_dir = tempfile.mkdtemp(prefix="llmc_b200_parity_")
    ref = subprocess.run([exe] + flags + ["-pn", "1", "-pr", "0", "-pg", "8", "-pi", "fs", "-pf", sync_dir], cwd=os.path.dirname(exe),
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=3000)
    if ref.returncode != 0:
        print("the reference trainer exited with code %d:\n%s" % (ref.returncode, ref.stdout[-2000:]))
        return 2
    ours = subprocess.run([sys.executable, os.path.join(ROOT, "train_gpt2.py")] + flags, cwd=ROOT, stdout=subprocess.PIPE,
                          stderr=subprocess.STDOUT, text=True, timeout=3000)
    if ours.returncode != 0:
        print("train_gpt2.py exited with code %d:\n%s" % (ours.returncode, ours.stdout[-2000:]))
        return 2
    lr, lo = losses_from(ref.stdout), losses_from(ours.stdout)
    n = min(len(lr), len(lo))
    if n < a.steps:
        print("parsed %d reference and %d own step lines, expected %d" % (len(lr), len(lo), a.steps))
        return 2
    print("step   reference        ours        diff")
    worst = 0.0
    for i in range(n):
        d = lo[i] - lr[i]
        worst = max(worst, abs(d))
        print("%4d   %9.6f   %9.6f   %+9.6f" % (i + 1, lr[i], lo[i], d))
    print("largest difference over %d steps: %.6f (tolerance %.3f)" % (n, worst, a.tol))
    return 0 if worst < a.tol else 1


if __name__ == "__main__":
    sys.exit(main())
