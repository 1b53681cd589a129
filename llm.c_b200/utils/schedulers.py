"""Learning-rate schedules cosine | linear | constant | wsd (reference: llmc/schedulers.h)."""
from . import _hostlib

TYPES = {"cosine": 0, "linear": 1, "constant": 2, "wsd": 3}


class LearningRateScheduler:
    def __init__(self, kind, learning_rate, warmup_iterations, train_num_batches, final_learning_rate_frac):
        if kind not in TYPES:
            raise ValueError("unknown learning rate scheduler type: %s" % kind)
        self.kind, self.learning_rate = kind, learning_rate
        self.warmup_iterations, self.train_num_batches = warmup_iterations, train_num_batches
        self.final_learning_rate_frac = final_learning_rate_frac
        self._lib = _hostlib.lib()

    def get_learning_rate(self, step):
        return float(self._lib.llmc_learning_rate(TYPES[self.kind], step, self.learning_rate, self.warmup_iterations,
                                                  self.train_num_batches, self.final_learning_rate_frac))
