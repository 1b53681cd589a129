"""Model checkpoints, per-rank optimizer/RNG state files and DONE markers, byte-compatible with the reference
(train_gpt2.cu:430-517 and 1209-1351 of the reference).

  model_%08d.bin        256 x int32 header {20240326, 3 (fp32) | 5 (bf16), maxT, V, L, NH, C, Vp}; parameters in flat order
  state_%08d_%05d.bin   256 x int32 header {20240527, 1, nproc, rank, use_master, shuffle, [10] step, [20:22] rng_state,
                        [22:24] rng_state_last_update, [30:32] shard idx, [32:34] sample idx}; m, v, (master) fp32 shards;
                        if shuffling: n_shards, shard_indices, n_samples, intra_shard_indices, raw mt19937 state
  DONE_%08d             empty marker, written by rank 0 once every rank has finished writing

Device tensors are streamed through a bounded pinned staging buffer, so writing a checkpoint needs no host copy of
the whole model.
"""
import os
import re
import struct

import numpy as np
import torch

from ..models.gpt2 import GPTConfig

MODEL_MAGIC, STATE_MAGIC = 20240326, 20240527
CHUNK_ELEMS = 16 * 1024 * 1024


def _stream_out(f, t):
    """Writes a (device or host) tensor to an open file in bounded chunks."""
    flat = t.reshape(-1)
    if flat.dtype == torch.bfloat16:
        flat = flat.view(torch.int16)
    for i in range(0, flat.numel(), CHUNK_ELEMS):
        f.write(flat[i:i + CHUNK_ELEMS].cpu().numpy().tobytes())


def _stream_in(f, t):
    """Fills a tensor from an open file in bounded chunks."""
    flat = t.reshape(-1)
    view = flat.view(torch.int16) if flat.dtype == torch.bfloat16 else flat
    np_dtype = {torch.int16: np.int16, torch.float32: np.float32, torch.int32: np.int32}[view.dtype]
    esz = view.element_size()
    for i in range(0, view.numel(), CHUNK_ELEMS):
        n = min(CHUNK_ELEMS, view.numel() - i)
        raw = f.read(n * esz)
        if len(raw) != n * esz:
            raise IOError("checkpoint file is truncated")
        view[i:i + n].copy_(torch.from_numpy(np.frombuffer(raw, dtype=np_dtype).copy()))


def write_model(path, model):
    cfg = model.cfg
    header = np.zeros(256, dtype=np.int32)
    version = 5 if model.dtype == torch.bfloat16 else 3
    header[:8] = [MODEL_MAGIC, version, cfg.max_seq_len, cfg.vocab_size, cfg.num_layers, cfg.num_heads, cfg.channels,
                  cfg.padded_vocab_size]
    with open(path, "wb") as f:
        f.write(header.tobytes())
        _stream_out(f, model.params_flat)


def read_model_header(path):
    with open(path, "rb") as f:
        header = np.frombuffer(f.read(1024), dtype=np.int32)
    if header.size != 256 or header[0] != MODEL_MAGIC:
        raise ValueError("bad magic in model file %s" % path)
    if header[1] not in (3, 5):
        raise ValueError("unsupported model file version %d (3 = fp32, 5 = bf16)" % header[1])
    cfg = GPTConfig(int(header[2]), int(header[3]), int(header[7]), int(header[4]), int(header[5]), int(header[6]))
    return cfg, int(header[1])


def load_model(path, model):
    """Loads parameters into an existing model (precision of the file may differ from the model's: values are cast)."""
    cfg, version = read_model_header(path)
    if cfg != model.cfg:
        raise ValueError("checkpoint %s does not match the model configuration" % path)
    file_dtype = torch.bfloat16 if version == 5 else torch.float32
    with open(path, "rb") as f:
        f.seek(1024)
        if file_dtype == model.dtype:
            _stream_in(f, model.params_flat)
        else:
            staging = torch.empty(CHUNK_ELEMS, dtype=file_dtype)
            flat = model.params_flat
            for i in range(0, flat.numel(), CHUNK_ELEMS):
                n = min(CHUNK_ELEMS, flat.numel() - i)
                _stream_in(f, staging[:n])
                flat[i:i + n].copy_(staging[:n])


def write_state(path, *, num_processes, process_rank, use_master_weights, step, rng_state, rng_state_last_update, m, v, master,
                loader):
    header = np.zeros(256, dtype=np.int32)
    header[0], header[1], header[2], header[3] = STATE_MAGIC, 1, num_processes, process_rank
    header[4] = 1 if use_master_weights else 0
    header[5] = 1 if loader.should_shuffle else 0
    header[10] = step
    shard_idx, sample_idx = loader.position()
    hb = bytearray(header.tobytes())
    struct.pack_into("<Q", hb, 20 * 4, rng_state & 0xFFFFFFFFFFFFFFFF)
    struct.pack_into("<Q", hb, 22 * 4, rng_state_last_update & 0xFFFFFFFFFFFFFFFF)
    struct.pack_into("<Q", hb, 30 * 4, shard_idx)
    struct.pack_into("<Q", hb, 32 * 4, sample_idx)
    with open(path, "wb") as f:
        f.write(bytes(hb))
        _stream_out(f, m)
        _stream_out(f, v)
        if use_master_weights:
            _stream_out(f, master)
        if loader.should_shuffle:
            shard_indices, intra, raw = loader.shuffle_state()
            f.write(struct.pack("<Q", shard_indices.size))
            f.write(shard_indices.astype(np.int32).tobytes())
            f.write(struct.pack("<Q", intra.size))
            f.write(intra.astype(np.int32).tobytes())
            f.write(raw)


def read_state(path, *, num_processes, process_rank, m, v, master, loader):
    """Fills m, v, (master) and restores the loader; returns dict(step, rng_state, rng_state_last_update, use_master_weights)."""
    with open(path, "rb") as f:
        hb = f.read(1024)
        header = np.frombuffer(hb, dtype=np.int32)
        if header[0] != STATE_MAGIC or header[1] != 1:
            raise ValueError("bad magic/version in state file %s" % path)
        if header[2] != num_processes or header[3] != process_rank:
            raise ValueError("state file %s was written by rank %d of %d" % (path, header[3], header[2]))
        use_master = bool(header[4])
        shuffled = bool(header[5])
        out = dict(step=int(header[10]), use_master_weights=use_master,
                   rng_state=struct.unpack_from("<Q", hb, 20 * 4)[0], rng_state_last_update=struct.unpack_from("<Q", hb, 22 * 4)[0])
        shard_idx = struct.unpack_from("<Q", hb, 30 * 4)[0]
        sample_idx = struct.unpack_from("<Q", hb, 32 * 4)[0]
        _stream_in(f, m)
        _stream_in(f, v)
        if use_master:
            if master is None:
                raise ValueError("state file has master weights but the run does not use them")
            _stream_in(f, master)
        if shuffled:
            (ns,) = struct.unpack("<Q", f.read(8))
            shard_indices = np.frombuffer(f.read(4 * ns), dtype=np.int32)
            (ni,) = struct.unpack("<Q", f.read(8))
            intra = np.frombuffer(f.read(4 * ni), dtype=np.int32)
            raw = f.read(2520)
            loader.set_shuffle_state(shard_indices, intra, raw)
        loader.resume(shard_idx, sample_idx)
    return out


def checkpoint_paths(log_dir, step, rank):
    return (os.path.join(log_dir, "model_%08d.bin" % step), os.path.join(log_dir, "state_%08d_%05d.bin" % (step, rank)),
            os.path.join(log_dir, "DONE_%08d" % step))


def find_max_step(log_dir):
    """Largest step with a DONE_ marker in log_dir, or -1 (reference: llmc/utils.h:192-210)."""
    best = -1
    if log_dir and os.path.isdir(log_dir):
        for name in os.listdir(log_dir):
            mt = re.fullmatch(r"DONE_(\d+)", name)
            if mt:
                best = max(best, int(mt.group(1)))
    return best


def delete_checkpoint(log_dir, step, rank):
    model, state, done = checkpoint_paths(log_dir, step, rank)
    for p in ([model, done] if rank == 0 else []) + [state]:
        try:
            os.remove(p)
        except FileNotFoundError:
            pass
