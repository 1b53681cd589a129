"""xorshift* random stream and softmax sampling (reference: llmc/sampler.h), backed by the C++ host runtime."""
import ctypes

from . import _hostlib


class Sampler:
    def __init__(self, seed=1337):
        self._lib = _hostlib.lib()
        self.state = ctypes.c_ulonglong(seed)

    def random_u32(self):
        return self._lib.llmc_random_u32(ctypes.byref(self.state))

    def random_f32(self):
        return self._lib.llmc_random_f32(ctypes.byref(self.state))

    def sample_softmax(self, logits, coin=None):
        """logits: 1-D float32 CPU tensor."""
        if coin is None:
            coin = self.random_f32()
        logits = logits.contiguous().float().cpu()
        return int(self._lib.llmc_sample_softmax(logits.data_ptr(), logits.numel(), coin))
