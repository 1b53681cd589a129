"""Buffers that live in device memory when it fits and in managed (host-resident) memory when it does not.

The optimizer state (two or three fp32 values per parameter of the local shard) is read and written once per step.  When the
device is full the trainer keeps it in managed memory whose preferred location is the host, so that a model that almost fits
still trains, at the cost of streaming that state over the host link during the update (capability parity with
cudaMallocConditionallyManaged of the reference, llmc/cuda_utils.cuh:213-229, used for the AdamW moments and the master
weights in train_gpt2.cu:1060-1085).  ``LLMC_FORCE_MANAGED=1`` takes the fallback unconditionally (tests).
"""
import ctypes
import os

import torch

_ITEM = {torch.float32: ("<f4", 4), torch.bfloat16: (None, 2), torch.int32: ("<i4", 4)}


class _Block:
    """Owns one allocation of the native runtime and exposes it to PyTorch through the CUDA array interface; the tensor made
    from it keeps this object, and with it the memory, alive."""

    def __init__(self, numel, dtype, force_managed):
        from .. import _lib
        typestr, size = _ITEM[dtype]
        if typestr is None:
            raise ValueError("managed buffers hold fp32 or int32")
        self._lib = _lib.cuda()
        ptr, managed = ctypes.c_void_p(), ctypes.c_int(0)
        _lib.check(self._lib.llmc_alloc_device_or_managed(ctypes.byref(ptr), numel * size, int(force_managed), ctypes.byref(managed)),
                   "llmc_alloc_device_or_managed")
        self.ptr, self.managed = ptr.value, bool(managed.value)
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (self.ptr, False), "version": 2, "strides": None}

    def __del__(self):
        ptr, self.ptr = getattr(self, "ptr", None), None
        if ptr:
            try:
                self._lib.llmc_free_device_or_managed(ctypes.c_void_p(ptr))
            except Exception:
                pass


def _device_zeros(numel, dtype, device):
    return torch.zeros(numel, dtype=dtype, device=device)


def _managed_zeros(numel, dtype, device, force):
    with torch.cuda.device(device):
        block = _Block(numel, dtype, force)
        t = torch.as_tensor(block, device=device)
    t.zero_()
    return t, block.managed


def zeros_device_or_managed(numel, dtype, device, what="buffer", log=print):
    """(tensor, managed).  On the host, or when the device has room, this is ``torch.zeros``."""
    device = torch.device(device)
    if device.type != "cuda":
        return torch.zeros(numel, dtype=dtype, device=device), False
    force = os.environ.get("LLMC_FORCE_MANAGED") == "1"
    if not force:
        try:
            return _device_zeros(numel, dtype, device), False
        except torch.cuda.OutOfMemoryError:
            torch.cuda.empty_cache()
    t, managed = _managed_zeros(numel, dtype, device, force)
    if managed and log is not None:
        log("%s: %.1f MiB placed in managed memory (device memory is exhausted); the optimizer step will be slower"
            % (what, numel * t.element_size() / 2 ** 20))
    return t, managed
