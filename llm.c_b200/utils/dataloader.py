"""Token-shard and evaluation-file loaders over the C++ host runtime, plus the writers of both formats.

Formats (identical to the reference, dev/data/data_common.py and llmc/dataloader.h):
  token shard  256 x int32 header {20240520, 1, ntok} followed by ntok x uint16, or {20240801, 7, ntok} followed by
               ntok x uint32 (LLaMA-3 vocabulary)
  eval file    256 x int32 header {20240522, 1, num_examples, longest_example_bytes} followed by, per example, the
               uint16 stream  65535, bytes, index, label, 4, ctx_len, ctx..., (len, tokens...) x 4

The training loader fills pinned int32 tensors; with ``prefetch=True`` the next batch is produced by a C++ worker
thread while the GPU works on the current one.  Rank r of n reads slot r of every global batch of n*B*T tokens.
"""
import ctypes
import struct

import numpy as np
import torch

from . import _hostlib
from .rand import STATE_BYTES


def write_datafile(path, tokens, model_desc="gpt-2"):
    """Token shard writer.  ``gpt-2``: ints < 65536 stored as uint16 (magic 20240520, version 1); ``llama-3``: uint32
    (magic 20240801, version 7), as the reference's dev/data/data_common.py:26-60 writes them."""
    if model_desc == "llama-3":
        arr = np.asarray(tokens, dtype=np.uint32)
        magic, version = 20240801, 7
    else:
        arr = np.asarray(tokens, dtype=np.uint16)
        magic, version = 20240520, 1
    header = np.zeros(256, dtype=np.int32)
    header[0], header[1], header[2] = magic, version, arr.size
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(arr.tobytes())


def write_synthetic_shard(path, ntok, vocab_size=50257, seed=0):
    """Seeded uniform-random uint16 tokens in [0, vocab_size): the synthetic data of the benchmarks."""
    rng = np.random.default_rng(seed)
    if vocab_size > 65536:
        write_datafile(path, rng.integers(0, vocab_size, size=ntok, dtype=np.uint32), "llama-3")
    else:
        write_datafile(path, rng.integers(0, vocab_size, size=ntok, dtype=np.uint16))


def write_evalfile(path, examples):
    """examples: list of dicts(ctx=[...], endings=[[...]]*4, label=int)."""
    header = np.zeros(256, dtype=np.int32)
    header[0], header[1], header[2] = 20240522, 1, len(examples)
    longest = 0
    blobs = []
    for idx, ex in enumerate(examples):
        stream = [ex["label"], len(ex["endings"]), len(ex["ctx"])] + list(ex["ctx"])
        for end in ex["endings"]:
            stream += [len(end)] + list(end)
        nbytes = (len(stream) + 3) * 2
        blob = struct.pack("<%dH" % (len(stream) + 3), 65535, nbytes, idx, *stream)
        longest = max(longest, nbytes)
        blobs.append(blob)
    header[3] = longest
    with open(path, "wb") as f:
        f.write(header.tobytes())
        for b in blobs:
            f.write(b)


def _pinned(shape, dtype):
    t = torch.empty(shape, dtype=dtype)
    if torch.cuda.is_available():
        try:
            t = t.pin_memory()
        except RuntimeError:
            pass
    return t


class DataLoader:
    def __init__(self, pattern, B, T, process_rank=0, num_processes=1, should_shuffle=False, prefetch=False):
        self._lib = _hostlib.lib()
        self.B, self.T = B, T
        self.process_rank, self.num_processes, self.should_shuffle = process_rank, num_processes, bool(should_shuffle)
        self._h = self._lib.llmc_dl_new(pattern.encode(), B, T, process_rank, num_processes, int(should_shuffle))
        if not self._h:
            raise _hostlib.HostError("DataLoader(%s): %s" % (pattern, _hostlib.last_error()))
        # two pinned buffer pairs so one can be filled while the other is being copied to the device
        self._bufs = [(_pinned((B, T), torch.int32), _pinned((B, T), torch.int32)) for _ in range(2)]
        self._cur = 0
        self._prefetch = prefetch
        self._inflight = False
        self.before_fill = None
        self.last_index = 0
        self.inputs, self.targets = self._bufs[0]

    def close(self):
        if getattr(self, "_h", None):
            self._lib.llmc_dl_free(self._h)
            self._h = None

    __del__ = close

    # properties read from the native object
    def _get(self, what):
        return int(self._lib.llmc_dl_get(self._h, what))

    num_tokens = property(lambda s: s._get(0))
    shard_num_samples = property(lambda s: s._get(1))
    current_shard_idx = property(lambda s: s._get(2))
    current_sample_idx = property(lambda s: s._get(3))
    num_shards = property(lambda s: s._get(4))

    def _drain(self):
        if self._inflight:
            _hostlib.check(self._lib.llmc_dl_wait(self._h), "DataLoader prefetch")
            self._inflight = False
            return True
        return False

    def next_batch(self):
        """Returns (inputs, targets): pinned int32 (B, T) tensors that stay valid until the call after next.
        ``before_fill(i)`` (if set) is called before buffer pair i is overwritten, ``last_index`` names the pair
        just returned: a caller that copies the batch to a device asynchronously records an event per pair after its
        copy and waits for it in ``before_fill``."""
        if self._prefetch:
            if not self._drain():       # first call: nothing in flight yet
                self._fill(self._cur, False)
            self.inputs, self.targets = self._bufs[self._cur]
            self.last_index = self._cur
            self._cur ^= 1
            self._fill(self._cur, True)
            self._inflight = True
        else:
            self._fill(self._cur, False)
            self.inputs, self.targets = self._bufs[self._cur]
            self.last_index = self._cur
            self._cur ^= 1
        return self.inputs, self.targets

    def _fill(self, idx, asynchronous):
        if self.before_fill is not None:
            self.before_fill(idx)
        i, t = self._bufs[idx]
        fn = self._lib.llmc_dl_prefetch if asynchronous else self._lib.llmc_dl_next
        _hostlib.check(fn(self._h, i.data_ptr(), t.data_ptr()), "DataLoader.next_batch")

    def reset(self):
        self._drain()
        _hostlib.check(self._lib.llmc_dl_reset(self._h), "DataLoader.reset")

    def resume(self, shard_idx, sample_idx):
        self._drain()
        _hostlib.check(self._lib.llmc_dl_resume(self._h, shard_idx, sample_idx), "DataLoader.resume")

    def position(self):
        """(shard index, sample index) of the next batch to be *returned* (a prefetched batch is not counted)."""
        s, i = self.current_shard_idx, self.current_sample_idx
        if self._inflight:
            self._drain()
            self._inflight = True      # result is still unread in the other buffer
            s, i = self.current_shard_idx, self.current_sample_idx - 1
        return s, i

    def shuffle_state(self):
        """(shard_indices, intra_shard_indices, raw mt19937 state) as stored in optimizer state files."""
        self._drain_keep()
        ns, ni = self.num_shards, self._get(5)
        a, b = np.zeros(ns, dtype=np.int32), np.zeros(max(ni, 1), dtype=np.int32)
        raw = ctypes.create_string_buffer(STATE_BYTES)
        self._lib.llmc_dl_get_shuffle_state(self._h, a.ctypes.data, b.ctypes.data, raw)
        return a, b[:ni], raw.raw

    def _drain_keep(self):
        if self._inflight:
            _hostlib.check(self._lib.llmc_dl_wait(self._h), "DataLoader prefetch")

    def set_shuffle_state(self, shard_indices, intra_indices, raw):
        self._drain()
        a = np.ascontiguousarray(shard_indices, dtype=np.int32)
        b = np.ascontiguousarray(intra_indices, dtype=np.int32)
        _hostlib.check(self._lib.llmc_dl_set_shuffle_state(self._h, a.ctypes.data, a.size, b.ctypes.data, b.size, ctypes.c_char_p(raw)),
                       "DataLoader.set_shuffle_state")


class EvalLoader:
    """Multiple-choice evaluation (HellaSwag format): four completions per example share one context."""

    def __init__(self, path, B, T, process_rank=0, num_processes=1):
        self._lib = _hostlib.lib()
        self.B, self.T = B, T
        self._h = self._lib.llmc_eval_new(path.encode(), B, T, process_rank, num_processes)
        if not self._h:
            raise _hostlib.HostError("EvalLoader(%s): %s" % (path, _hostlib.last_error()))
        self.inputs = _pinned((B, T), torch.int32).zero_()
        self.targets = _pinned((B, T), torch.int32).zero_()
        self.mask = torch.zeros(B, T, dtype=torch.int8)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.llmc_eval_free(self._h)
            self._h = None

    __del__ = close

    num_examples = property(lambda s: s._lib.llmc_eval_get(s._h, 0))
    num_batches = property(lambda s: s._lib.llmc_eval_get(s._h, 1))
    start_example_index = property(lambda s: s._lib.llmc_eval_get(s._h, 2))
    end_example_index = property(lambda s: s._lib.llmc_eval_get(s._h, 3))

    def reset(self):
        _hostlib.check(self._lib.llmc_eval_reset(self._h), "EvalLoader.reset")

    def next_batch(self):
        _hostlib.check(self._lib.llmc_eval_next_batch(self._h, self.inputs.data_ptr(), self.targets.data_ptr(), self.mask.data_ptr()),
                       "EvalLoader.next_batch")
        return self.inputs, self.targets, self.mask

    def stat_losses(self, losses):
        """losses: float32 CPU tensor (B, T) of per-token losses; returns the number of correct examples in the batch."""
        losses = losses.contiguous().float().cpu()
        return int(self._lib.llmc_eval_stat_losses(self._h, losses.data_ptr(), self.mask.data_ptr()))
