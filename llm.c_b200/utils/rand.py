"""mt19937 random numbers, bit-identical to PyTorch's CPU generator (reference: llmc/rand.h).

Used for parameter initialisation and data shuffling so that runs can be compared with, and resumed
from, files produced by the reference."""
import ctypes

import torch

from . import _hostlib

STATE_BYTES = 2520


class MT19937:
    def __init__(self, seed=5489):
        self._lib = _hostlib.lib()
        self._h = self._lib.llmc_rng_new(seed & 0xFFFFFFFF)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.llmc_rng_free(self._h)
            self._h = None

    def randint32(self):
        return self._lib.llmc_rng_u32(self._h)

    def randfloat32(self):
        return self._lib.llmc_rng_f32(self._h)

    def uniform(self, n, lo=0.0, hi=1.0):
        out = torch.empty(n, dtype=torch.float32)
        self._lib.llmc_rng_uniform(self._h, out.data_ptr(), n, lo, hi)
        return out

    def normal(self, n, mean=0.0, std=1.0):
        out = torch.empty(n, dtype=torch.float32)
        self._lib.llmc_rng_normal(self._h, out.data_ptr(), n, mean, std)
        return out

    def permutation(self, n):
        out = torch.arange(n, dtype=torch.int32)
        self._lib.llmc_rng_permutation(self._h, out.data_ptr(), n)
        return out

    def get_state(self):
        buf = ctypes.create_string_buffer(STATE_BYTES)
        self._lib.llmc_rng_get_state(self._h, buf)
        return buf.raw

    def set_state(self, raw):
        assert len(raw) == STATE_BYTES
        self._lib.llmc_rng_set_state(self._h, ctypes.c_char_p(raw))
