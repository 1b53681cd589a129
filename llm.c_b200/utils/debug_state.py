"""GPT-2 debug-state file: one batch with the logits, loss and gradients a model must reproduce on it.

Layout of the reference (writer train_gpt2.py:479-507, readers test_gpt2.c:60-86 and test_gpt2.cu:127-160 of the
reference): 256 x int32 header {20240327, 2, B, T}; x int32[B*T]; y int32[B*T]; logits fp32[B*T*V] (unpadded
vocabulary); loss fp32; the gradients of all 16 parameter tensors in file order as fp32, the token embedding padded
with zero rows to the padded vocabulary.

``write_debug_state`` fills the file from any source of (logits, loss, gradients): the autograd oracle of the tests, or
a model of this framework itself (``from_model``), which then serves as the golden record for another precision or
device.  ``read_debug_state`` returns the fields; ``check_model`` runs a model on the stored batch and reports the
largest deviations, the way the reference's test programs do.

    python -m llmc_b200.utils.debug_state -e d12 -b 4 -t 64 -o gpt2_124M_debug_state.bin [-m gpt2_124M.bin]
"""
import numpy as np
import torch

from ..models.gpt2 import PARAM_NAMES, param_shapes

MAGIC, VERSION = 20240327, 2


def write_debug_state(path, cfg, x, y, logits, loss, grads):
    """x, y: (B, T) integer tensors; logits: (B, T, >= V) floats (extra columns are dropped); grads: name -> tensor."""
    B, T = x.shape
    V, Vp = cfg.vocab_size, cfg.padded_vocab_size
    header = np.zeros(256, dtype=np.int32)
    header[:4] = [MAGIC, VERSION, B, T]
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(x.cpu().numpy().astype(np.int32).tobytes())
        f.write(y.cpu().numpy().astype(np.int32).tobytes())
        f.write(logits[..., :V].float().cpu().contiguous().numpy().tobytes())
        f.write(np.float32(loss).tobytes())
        for name, shape in param_shapes(cfg):
            g = grads[name].float().cpu().reshape(shape)
            if name == "wte" and g.shape[0] != Vp:          # a source with an unpadded embedding: pad with zero rows
                g = torch.cat([g, torch.zeros(Vp - g.shape[0], g.shape[1])])
            f.write(g.contiguous().numpy().tobytes())


def from_model(path, model, x, y):
    """Runs ``model`` on the batch and stores what it computed."""
    model.forward(x.to(model.device), y.to(model.device), write_dlogits=False)
    logits = model.logits().float().cpu().clone()
    model.forward(x.to(model.device), y.to(model.device))
    model.backward()
    write_debug_state(path, model.cfg, x, y, logits, float(model.loss()), {n: model.grads[n] for n in PARAM_NAMES})


def read_debug_state(path, cfg):
    """Returns dict(B, T, x, y, logits (B, T, V), loss, grads {name: tensor in parameter shape})."""
    V = cfg.vocab_size
    with open(path, "rb") as f:
        header = np.frombuffer(f.read(1024), dtype=np.int32)
        if header.size != 256 or header[0] != MAGIC:
            raise ValueError("bad magic in debug-state file %s" % path)
        if header[1] != VERSION:
            raise ValueError("unsupported debug-state version %d (expected %d)" % (header[1], VERSION))
        B, T = int(header[2]), int(header[3])

        def take(n, dtype):
            raw = f.read(n * np.dtype(dtype).itemsize)
            if len(raw) != n * np.dtype(dtype).itemsize:
                raise IOError("debug-state file %s is truncated" % path)
            return torch.from_numpy(np.frombuffer(raw, dtype=dtype).copy())

        x = take(B * T, np.int32).view(B, T)
        y = take(B * T, np.int32).view(B, T)
        logits = take(B * T * V, np.float32).view(B, T, V)
        loss = float(take(1, np.float32)[0])
        grads = {}
        for name, shape in param_shapes(cfg):
            n = int(np.prod(shape))
            grads[name] = take(n, np.float32).view(shape)
        if f.read(1):
            raise ValueError("debug-state file %s is longer than its header implies" % path)
    return dict(B=B, T=T, x=x, y=y, logits=logits, loss=loss, grads=grads)


def check_model(model, state):
    """Forward and backward of ``model`` on the stored batch; returns dict(logits, loss, grads {name: max abs deviation})."""
    x, y = state["x"].to(model.device), state["y"].to(model.device)
    V = model.cfg.vocab_size
    model.forward(x, y, write_dlogits=False)
    dev_logits = (model.logits()[..., :V].float().cpu() - state["logits"]).abs().max().item()
    model.forward(x, y)
    model.backward()
    out = dict(logits=dev_logits, loss=abs(float(model.loss()) - state["loss"]), grads={})
    for name in PARAM_NAMES:
        out["grads"][name] = (model.grads[name].float().cpu() - state["grads"][name]).abs().max().item()
    return out


def main(argv=None):
    import argparse
    from ..models import gpt2
    from . import checkpoint
    ap = argparse.ArgumentParser(description="write a model file and its debug state from a random-init or loaded GPT-2")
    ap.add_argument("-e", default="d12", help="descriptor (d12, gpt3:c768) or model file")
    ap.add_argument("-b", type=int, default=4)
    ap.add_argument("-t", type=int, default=64)
    ap.add_argument("-o", default="gpt2_124M_debug_state.bin")
    ap.add_argument("-m", default="", help="also write the model file here (fp32, version 3)")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.e.endswith(".bin"):
        cfg, _ = checkpoint.read_model_header(a.e)
        model = gpt2.GPT(cfg, "cpu", torch.float32, recompute=0)
        checkpoint.load_model(a.e, model)
    else:
        model = gpt2.GPT(gpt2.config_from_descriptor(a.e), "cpu", torch.float32, recompute=0)
        model.init_random(42)
    g = torch.Generator().manual_seed(a.seed)
    tok = torch.randint(0, model.cfg.vocab_size, (a.b, a.t + 1), generator=g, dtype=torch.int32)
    from_model(a.o, model, tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
    if a.m:
        checkpoint.write_model(a.m, model)
    print("wrote %s" % a.o)
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
