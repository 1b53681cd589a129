"""Model checkpoints, per-rank optimizer/RNG state files and DONE markers, byte-compatible with the reference
(train_gpt2.cu:430-517 and 1209-1351 of the reference).

  model_%08d.bin        256 x int32 header {20240326, 3 (fp32) | 5 (bf16), maxT, V, L, NH, C, Vp}; parameters in flat order
  state_%08d_%05d.bin   256 x int32 header {20240527, 1, nproc, rank, use_master, shuffle, [10] step, [20:22] rng_state,
                        [22:24] rng_state_last_update, [30:32] shard idx, [32:34] sample idx}; m, v, (master) fp32 shards;
                        if shuffling: n_shards, shard_indices, n_samples, intra_shard_indices, raw mt19937 state
  DONE_%08d             empty marker, written by rank 0 once every rank has finished writing

LLaMA-3 models use the reference's own header and tensor order (train_llama3.py:851-905 of the reference):
  header {20240803, 3 | 5, block_size, vocab_size, n_layer, n_head, n_kv_head, n_embd, int(ffn_dim_multiplier), multiple_of,
  int(norm_eps), int(rope_theta), use_scaled_rope, max_gen_batch_size, version major, version minor}; tensors wte, ln_1, c_attn,
  attn c_proj, ln_2, c_fc, c_fc2, mlp c_proj, ln_f, lm_head, each stacked over layers.  The reference's writer truncates the
  three float fields to integers; this writer also stores them exactly, as three float64 in header[17:23] (marker 1 in
  header[16]), and the padded vocabulary in header[23]; the reference's readers ignore those slots.

Device tensors are streamed through two pinned staging buffers (transfer and file IO overlap), so writing or reading a
checkpoint needs no host copy of the whole model.
"""
import os
import re
import struct

import numpy as np
import torch

from ..models.gpt2 import GPTConfig

MODEL_MAGIC, STATE_MAGIC, LLAMA_MAGIC = 20240326, 20240527, 20240803
CHUNK_ELEMS = 16 * 1024 * 1024


class _atomic_write:
    """Opens ``path + '.tmp'`` for writing and renames it onto ``path`` when the block ends without an exception: a process killed
    in the middle of a checkpoint leaves no truncated file under the final name (the restart loop would load it)."""

    def __init__(self, path):
        self.path, self.tmp, self.f = path, path + ".tmp", None

    def __enter__(self):
        self.f = open(self.tmp, "wb")
        return self.f

    def __exit__(self, exc_type, exc, tb):
        self.f.flush()
        os.fsync(self.f.fileno())
        self.f.close()
        if exc_type is None:
            os.replace(self.tmp, self.path)
        else:
            try:
                os.remove(self.tmp)
            except OSError:
                pass
        return False


_staging = {}


def _pinned_pair(dtype):
    """Two pinned host buffers of CHUNK_ELEMS elements per element type, allocated once (reference: the double buffer of
    device_to_file / file_to_device in llmc/cuda_common.h)."""
    if dtype not in _staging:
        _staging[dtype] = [torch.empty(CHUNK_ELEMS, dtype=dtype).pin_memory() for _ in range(2)]
    return _staging[dtype]


def _raw_view(t):
    flat = t.reshape(-1)
    return flat.view(torch.int16) if flat.dtype == torch.bfloat16 else flat


def _stream_out(f, t):
    """Writes a tensor to an open file.  Host tensors go out through their buffer, without a copy.  Device tensors are staged
    through two pinned buffers: while chunk i is written to the file, the copy of chunk i + 1 is already running on a side
    stream, so the device-to-host transfer and the file write overlap and no host copy of the whole tensor ever exists."""
    view = _raw_view(t)
    n_total = view.numel()
    if n_total == 0:
        return
    if not view.is_cuda:
        f.write(memoryview(view.contiguous().numpy()).cast("B"))
        return
    bufs = _pinned_pair(view.dtype)
    side = torch.cuda.Stream(device=view.device)
    side.wait_stream(torch.cuda.current_stream(view.device))       # whatever produced the tensor has finished
    events = [torch.cuda.Event(), torch.cuda.Event()]

    def start(chunk):
        i = chunk * CHUNK_ELEMS
        n = min(CHUNK_ELEMS, n_total - i)
        with torch.cuda.stream(side):
            bufs[chunk & 1][:n].copy_(view[i:i + n], non_blocking=True)
            events[chunk & 1].record(side)
        return n

    chunks = (n_total + CHUNK_ELEMS - 1) // CHUNK_ELEMS
    pending = start(0)
    for c in range(chunks):
        n = pending
        if c + 1 < chunks:
            pending = start(c + 1)            # the other buffer: its previous contents were written in the last trip
        events[c & 1].synchronize()
        f.write(memoryview(bufs[c & 1][:n].numpy()).cast("B"))


def _stream_in(f, t):
    """Fills a tensor from an open file.  Device tensors: the file is read into one pinned buffer while the host-to-device copy
    of the previous chunk runs from the other."""
    view = _raw_view(t)
    n_total = view.numel()
    esz = view.element_size()
    if not t.is_contiguous():
        raise ValueError("checkpoint tensors must be contiguous")
    if not view.is_cuda:
        got = f.readinto(memoryview(view.numpy()).cast("B")) if n_total else 0
        if got != n_total * esz:
            raise IOError("checkpoint file is truncated")
        return
    bufs = _pinned_pair(view.dtype)
    events = [None, None]
    stream = torch.cuda.current_stream(view.device)
    for c, i in enumerate(range(0, n_total, CHUNK_ELEMS)):
        n = min(CHUNK_ELEMS, n_total - i)
        if events[c & 1] is not None:
            events[c & 1].synchronize()       # the copy that last read this buffer has finished
        got = f.readinto(memoryview(bufs[c & 1][:n].numpy()).cast("B"))
        if got != n * esz:
            raise IOError("checkpoint file is truncated")
        view[i:i + n].copy_(bufs[c & 1][:n], non_blocking=True)
        events[c & 1] = torch.cuda.Event()
        events[c & 1].record(stream)
    for e in events:
        if e is not None:
            e.synchronize()                   # the staging buffers are shared: leave them idle


def write_model(path, model):
    if getattr(model, "family", "gpt2") == "llama3":
        return _write_llama(path, model)
    cfg = model.cfg
    header = np.zeros(256, dtype=np.int32)
    version = 5 if model.dtype == torch.bfloat16 else 3
    header[:8] = [MODEL_MAGIC, version, cfg.max_seq_len, cfg.vocab_size, cfg.num_layers, cfg.num_heads, cfg.channels,
                  cfg.padded_vocab_size]
    with _atomic_write(path) as f:
        f.write(header.tobytes())
        _stream_out(f, model.params_flat)


def model_family(path):
    """'gpt2' or 'llama3', from the magic number of a model file."""
    with open(path, "rb") as f:
        magic = np.frombuffer(f.read(4), dtype=np.int32)
    if magic.size == 1 and magic[0] == LLAMA_MAGIC:
        return "llama3"
    return "gpt2"


def read_model_header(path):
    with open(path, "rb") as f:
        header = np.frombuffer(f.read(1024), dtype=np.int32)
    if header.size == 256 and header[0] == LLAMA_MAGIC:
        return _read_llama_header(header, path)
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
    if getattr(model, "family", "gpt2") == "llama3":
        return _load_llama(path, model, file_dtype)
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


# ---------------------------------------------------------------------------------------------------------------
# LLaMA-3 model files

def _llama_file_tensors(model):
    """The tensors of a LLaMA model in file order, as lists of flat-buffer views that are contiguous in memory: the fused
    up-projection (L, 2H, C) is split into its c_fc rows (all layers) followed by its c_fc2 rows (all layers)."""
    p, L, H = model.params, model.cfg.num_layers, model.cfg.hidden_dim
    out = []
    for name in ("wte", "ln1w", "qkvw", "attprojw", "ln2w"):
        out.append(p[name])
    out += [p["fc12w"][l, :H] for l in range(L)]
    out += [p["fc12w"][l, H:] for l in range(L)]
    for name in ("fcprojw", "lnfw", "lmhead"):
        out.append(p[name])
    return out


def _write_llama(path, model):
    cfg = model.cfg
    header = np.zeros(256, dtype=np.int32)
    version = 5 if model.dtype == torch.bfloat16 else 3
    major, minor = (int(x) for x in cfg.version.split("."))
    header[:16] = [LLAMA_MAGIC, version, cfg.max_seq_len, cfg.vocab_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads,
                   cfg.channels, int(cfg.ffn_dim_multiplier), cfg.multiple_of, int(cfg.norm_eps), int(cfg.rope_theta),
                   int(cfg.use_scaled_rope), 4, major, minor]
    header[16] = 1
    header[17:23] = np.array([cfg.ffn_dim_multiplier, cfg.norm_eps, cfg.rope_theta], dtype=np.float64).view(np.int32)
    header[23] = cfg.padded_vocab_size
    Vp, V = cfg.padded_vocab_size, cfg.vocab_size
    with _atomic_write(path) as f:
        f.write(header.tobytes())
        for t in _llama_file_tensors(model):
            if t.shape[0] == Vp and t.dim() == 2 and Vp != V:
                t = t[:V]                      # files hold the unpadded vocabulary, like the reference's
            _stream_out(f, t)


def _read_llama_header(header, path):
    from ..models.llama3 import LlamaConfig, _pad128
    if header[1] not in (3, 5):
        raise ValueError("unsupported model file version %d (3 = fp32, 5 = bf16)" % header[1])
    if header[16] == 1:
        ffn, eps, theta = (float(x) for x in np.ascontiguousarray(header[17:23]).view(np.float64))
        vp = int(header[23])
    else:
        # a file from the reference's writer: the float fields were truncated to integers; LLaMA-3.1 values
        ffn, eps, theta, vp = (1.2 if header[7] == 16384 else 1.3), 1e-5, float(header[11]), _pad128(int(header[3]))
    cfg = LlamaConfig(max_seq_len=int(header[2]), vocab_size=int(header[3]), padded_vocab_size=vp, num_layers=int(header[4]),
                      num_heads=int(header[5]), num_kv_heads=int(header[6]), channels=int(header[7]), ffn_dim_multiplier=ffn,
                      multiple_of=int(header[9]), norm_eps=eps, rope_theta=theta, use_scaled_rope=bool(header[12]),
                      version="%d.%d" % (header[14], header[15]))
    return cfg, int(header[1])


def _load_llama(path, model, file_dtype):
    cfg = model.cfg
    Vp, V = cfg.padded_vocab_size, cfg.vocab_size
    staging = None if file_dtype == model.dtype else torch.empty(CHUNK_ELEMS, dtype=file_dtype)
    with open(path, "rb") as f:
        f.seek(1024)
        for t in _llama_file_tensors(model):
            if t.shape[0] == Vp and t.dim() == 2 and Vp != V:
                t[V:].zero_()
                t = t[:V]
            flat = t.reshape(-1)               # a view: every listed tensor is contiguous in the flat buffer
            if staging is None:
                _stream_in(f, flat)
            else:
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
    with _atomic_write(path) as f:
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
