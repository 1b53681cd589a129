"""``main.log`` writer (rank 0 only) in the line format of the reference (llmc/logger.h:34-56), so its log
visualiser parses our runs, plus an optional JSON-lines stream with device timings."""
import json
import os


class Logger:
    def __init__(self, log_dir, process_rank=0, resume=False):
        self.active = bool(log_dir) and process_rank == 0
        self.path = None
        self.jsonl = None
        if self.active:
            os.makedirs(log_dir, exist_ok=True)
            self.path = os.path.join(log_dir, "main.log")
            self.jsonl = os.path.join(log_dir, "metrics.jsonl")
            if not resume:
                open(self.path, "w").close()
                open(self.jsonl, "w").close()

    def _append(self, line):
        if self.active:
            with open(self.path, "a") as f:
                f.write(line + "\n")

    def log_val(self, step, val_loss):
        self._append("s:%d tel:%.4f" % (step, val_loss))

    def log_eval(self, step, val):
        self._append("s:%d eval:%.4f" % (step, val))

    def log_train(self, step, train_loss, learning_rate, grad_norm):
        self._append("s:%d trl:%.4f lr:%.6f norm:%.2f" % (step, train_loss, learning_rate, grad_norm))

    def log_metrics(self, **kv):
        if self.active:
            with open(self.jsonl, "a") as f:
                f.write(json.dumps(kv) + "\n")
