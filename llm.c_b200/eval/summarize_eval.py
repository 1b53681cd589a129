"""Prints the six benchmark scores of one evaluation-harness result folder and their average
(reference: dev/eval/summarize_eval.py; the folder is what ``run_eval.sh`` beside this file writes).

    python -m llmc_b200.eval.summarize_eval lm-evaluation-harness/results/my_run
"""
import json
import os
import sys

# result file -> the metric the leaderboard reads from it
TASKS = [("arc_challenge_25shot.json", "acc_norm"), ("gsm8k_5shot.json", "acc"), ("hellaswag_10shot.json", "acc_norm"),
         ("mmlu_5shot.json", "acc"), ("truthfulqa_0shot.json", "mc2"), ("winogrande_5shot.json", "acc")]


def summarize(result_dir, out=sys.stdout):
    """Returns {file: score in percent} (mean over the sub-tasks of a file) and prints the table; a missing file is reported
    and left out of the average instead of ending the run."""
    scores = {}
    print("-" * 40, file=out)
    for fname, key in TASKS:
        path = os.path.join(result_dir, fname)
        try:
            with open(path) as f:
                results = json.load(f)["results"]
        except (OSError, ValueError, KeyError) as e:
            print("%-30s : missing (%s)" % (fname, type(e).__name__), file=out)
            continue
        vals = [r[key] for r in results.values() if key in r]
        if not vals:
            print("%-30s : no '%s' entries" % (fname, key), file=out)
            continue
        scores[fname] = 100.0 * sum(vals) / len(vals)
        print("%-30s : %.4f" % (fname, scores[fname]), file=out)
    print("-" * 40, file=out)
    if scores:
        print("%-30s : %.4f  (%d of %d tasks)" % ("Average Score", sum(scores.values()) / len(scores), len(scores), len(TASKS)), file=out)
    return scores


if __name__ == "__main__":
    if len(sys.argv) != 2:
        print(__doc__)
        sys.exit(1)
    summarize(sys.argv[1])
