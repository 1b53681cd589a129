"""GPT-2 / GPT-3 style decoder on flat parameter and gradient buffers.

The model owns one contiguous parameter buffer and one gradient buffer laid out in the order of the
reference's checkpoint files (train_gpt2.cu:118-144 of the reference: wte wpe ln1w ln1b qkvw qkvb
attprojw attprojb ln2w ln2b fcw fcb fcprojw fcprojb lnfw lnfb, per-layer tensors stacked over L) and
all activations of a (B, T) micro-batch, allocated once.  Forward and backward are written out by
hand on top of ``ops`` (no autograd): on a GPU every call is one of this library's sm_100a kernels, on
the CPU the same code runs on the PyTorch fp32 restatement, which is the counterpart of the
reference's train_gpt2.c.

Differences from the reference's schedule that matter for speed on a B200:
  * GELU forward and its derivative run inside the GEMM epilogues; no separate passes.
  * Gradients are written (not added) on the first micro-step, so no gradient memset per step.
  * The backward pass performs no host synchronisation; the loss is read once per step.
  * Token/position gradient bucketing happens on the device (see csrc/encoder.cu).
"""
import math
from dataclasses import dataclass

import torch

from .. import ops


class _Range:
    """NVTX range on CUDA devices (the reference's NvtxRange, llmc/cuda_common.h:115-124); a no-op elsewhere."""

    def __init__(self, name, on):
        self.name, self.on = name, on

    def __enter__(self):
        if self.on:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()

PARAM_NAMES = ["wte", "wpe", "ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb", "ln2w", "ln2b", "fcw", "fcb",
               "fcprojw", "fcprojb", "lnfw", "lnfb"]
# tensors that receive weight decay (2-D weights): reference train_gpt2.cu:1080
DECAYED = {"wte", "wpe", "qkvw", "attprojw", "fcw", "fcprojw"}
LAYERED = set(PARAM_NAMES[2:14])


@dataclass
class GPTConfig:
    max_seq_len: int = 1024
    vocab_size: int = 50257
    padded_vocab_size: int = 50304
    num_layers: int = 12
    num_heads: int = 12
    channels: int = 768

    @property
    def head_size(self):
        return self.channels // self.num_heads


def gpt2_descriptor(depth):
    """GPT-2 family by depth (reference train_gpt2.cu:519-536)."""
    table = {6: (384, 6), 12: (768, 12), 24: (1024, 16), 36: (1280, 20), 48: (1600, 25), 60: (1920, 30), 72: (2880, 30),
             84: (3456, 36)}
    if depth not in table:
        raise ValueError("unsupported GPT-2 depth %d" % depth)
    c, nh = table[depth]
    return GPTConfig(1024, 50257, 50304, depth, nh, c)


def gpt3_descriptor(channels):
    """GPT-3 family by width (reference train_gpt2.cu:538-560); context 2048."""
    # width -> (depth, head size); the number of heads follows
    table = {384: (6, 64), 768: (12, 64), 1024: (24, 64), 1536: (24, 96), 2048: (24, 128), 2560: (32, 80), 4096: (32, 128),
             5140: (40, 128), 12288: (96, 128)}
    if channels not in table:
        raise ValueError("unsupported GPT-3 width %d" % channels)
    L, hs = table[channels]
    if channels % hs:
        raise ValueError("GPT-3 width %d is not divisible by its head size %d" % (channels, hs))
    nh = channels // hs
    return GPTConfig(2048, 50257, 50304, L, nh, channels)


def config_from_descriptor(desc):
    """'d12', 'gpt2:d12' or 'gpt3:c768'."""
    if desc.startswith("gpt2:"):
        desc = desc[5:]
    if desc.startswith("gpt3:"):
        body = desc[5:]
        if not body.startswith("c"):
            raise ValueError("GPT-3 descriptor must look like gpt3:c768")
        return gpt3_descriptor(int(body[1:]))
    if desc.startswith("d"):
        return gpt2_descriptor(int(desc[1:]))
    raise ValueError("unknown model descriptor %r" % desc)


def param_shapes(cfg):
    L, C, Vp, maxT = cfg.num_layers, cfg.channels, cfg.padded_vocab_size, cfg.max_seq_len
    return [("wte", (Vp, C)), ("wpe", (maxT, C)), ("ln1w", (L, C)), ("ln1b", (L, C)), ("qkvw", (L, 3 * C, C)),
            ("qkvb", (L, 3 * C)), ("attprojw", (L, C, C)), ("attprojb", (L, C)), ("ln2w", (L, C)), ("ln2b", (L, C)),
            ("fcw", (L, 4 * C, C)), ("fcb", (L, 4 * C)), ("fcprojw", (L, C, 4 * C)), ("fcprojb", (L, C)), ("lnfw", (C,)),
            ("lnfb", (C,))]


def num_parameters(cfg):
    return sum(math.prod(s) for _, s in param_shapes(cfg))


class GPT:
    family = "gpt2"
    norm_params = ("ln1w", "ln1b", "ln2w", "ln2b")      # per-layer tensors that the forward pass reads before the layer's first GEMM

    def __init__(self, cfg, device="cpu", dtype=None, recompute=1, flat_allocator=None):
        """``flat_allocator(kind, numel, dtype)`` (kind = 'params' | 'grads') may supply the two flat buffers, e.g. from
        symmetric memory that peer GPUs can address; by default they are ordinary tensors."""
        self.cfg = cfg
        self.device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("parameters are bf16 (sm_100a kernels) or fp32 (full-precision mode)")
        if cfg.channels % 8 or (self.device.type == "cuda" and dtype == torch.bfloat16 and (cfg.head_size % 8 or not 64 <= cfg.head_size <= 128)):
            raise ValueError("channels must be a multiple of 8 and (on the GPU) the head size a multiple of 8 from 64 to 128")
        self.dtype = dtype
        self.recompute = recompute
        self.shapes = param_shapes(cfg)
        self.num_parameters = num_parameters(cfg)
        self.offsets = {}
        off = 0
        for name, shape in self.shapes:
            self.offsets[name] = off
            off += math.prod(shape)
        self._flat_allocator = flat_allocator
        if flat_allocator is not None:
            self.params_flat = flat_allocator("params", self.num_parameters, dtype)
        else:
            self.params_flat = torch.zeros(self.num_parameters, dtype=dtype, device=self.device)
        self.grads_flat = None
        self.params = self._views(self.params_flat)
        self.grads = None
        self.acts = None
        self.act_shape = None
        self.inputs = None
        self.targets = None
        self.mean_loss = None          # device scalar after a backward with targets
        self.grad_hook = None
        # set by a communication backend whose all-gather may still be in flight when forward starts (parallel/p2p.py)
        self.param_sync = None          # called as grad_hook(layer or -1 for the embeddings/final LN) on the last micro-step

    # ------------------------------------------------------------------ parameters
    def _views(self, flat):
        out = {}
        for name, shape in self.shapes:
            o = self.offsets[name]
            out[name] = flat[o:o + math.prod(shape)].view(shape)
        return out

    def tensor_sizes(self):
        """(name, offset, per-layer size, number of layer slices) for every parameter tensor."""
        res = []
        for name, shape in self.shapes:
            n = math.prod(shape)
            L = self.cfg.num_layers if name in LAYERED else 1
            res.append((name, self.offsets[name], n // L, L))
        return res

    def init_random(self, seed=42, generator_factory=None):
        """GPT-2 initialisation in the draw order of the reference (train_gpt2.cu:587-642): one normal stream,
        layer by layer; std 0.02, residual projections 0.02/sqrt(2L); LayerNorm weights 1; biases 0."""
        from ..utils import rand
        cfg = self.cfg
        rng = rand.MT19937(seed)
        host = {n: torch.zeros(s, dtype=torch.float32) for n, s in self.shapes}
        for n in ("ln1w", "ln2w", "lnfw"):
            host[n].fill_(1.0)
        resid_std = 0.02 / math.sqrt(2.0 * cfg.num_layers)
        for l in range(cfg.num_layers):
            if l == 0:
                host["wte"][:cfg.vocab_size] = rng.normal(cfg.vocab_size * cfg.channels, 0.0, 0.02).view(cfg.vocab_size, cfg.channels)
                host["wpe"].copy_(rng.normal(cfg.max_seq_len * cfg.channels, 0.0, 0.02).view(cfg.max_seq_len, cfg.channels))
            for n, std in (("qkvw", 0.02), ("attprojw", resid_std), ("fcw", 0.02), ("fcprojw", resid_std)):
                host[n][l] = rng.normal(host[n][l].numel(), 0.0, std).view(host[n][l].shape)
        for n, _ in self.shapes:
            self.params[n].copy_(host[n])

    # ------------------------------------------------------------------ buffers
    def allocate_grads(self):
        if self.grads_flat is None:
            if self._flat_allocator is not None:
                self.grads_flat = self._flat_allocator("grads", self.num_parameters, self.dtype)
            else:
                self.grads_flat = torch.zeros(self.num_parameters, dtype=self.dtype, device=self.device)
            self.grads = self._views(self.grads_flat)

    def allocate_activations(self, B, T):
        if self.act_shape == (B, T):
            return
        cfg, dev, dt = self.cfg, self.device, self.dtype
        L, C, NH, Vp = cfg.num_layers, cfg.channels, cfg.num_heads, cfg.padded_vocab_size
        N = B * T
        Lln = 1 if self.recompute >= 2 else L
        Lg = 1 if self.recompute >= 1 else L
        e = lambda *s, dtype=dt: torch.empty(*s, dtype=dtype, device=dev)
        f32 = torch.float32
        self.acts = dict(
            encoded=e(N, C), ln1=e(Lln, N, C), ln1_mean=e(L, N, dtype=f32), ln1_rstd=e(L, N, dtype=f32),
            qkv=e(L, N, 3 * C), atty=e(L, N, C), lse=e(L, B, NH, T, dtype=f32), residual2=e(L, N, C),
            ln2=e(Lln, N, C), ln2_mean=e(L, N, dtype=f32), ln2_rstd=e(L, N, dtype=f32), fch=e(L, N, 4 * C),
            fch_gelu=e(Lg, N, 4 * C), residual3=e(L, N, C), lnf=e(N, C), lnf_mean=e(N, dtype=f32), lnf_rstd=e(N, dtype=f32),
            losses=torch.zeros(N, dtype=f32, device=dev), logits=e(N, Vp), scratch_btc=e(N, C), scratch_bt4c=e(N, 4 * C),
            dresidual=e(N, C), dqkv=e(N, 3 * C),
        )
        self.inputs = torch.zeros(B, T, dtype=torch.int32, device=dev)
        self.targets = torch.zeros(B, T, dtype=torch.int32, device=dev)
        self.mean_loss = torch.zeros(1, dtype=f32, device=dev)
        self.act_shape = (B, T)

    def activation_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.acts.values()) if self.acts else 0

    # ------------------------------------------------------------------ forward
    def forward(self, tokens, targets=None, grad_accum_steps=1, micro_step=0, write_dlogits=True):
        """Runs the network on tokens (B, T) int32.  With targets, the per-token losses are accumulated into
        ``acts['losses']`` and (if write_dlogits) the logits buffer is turned into dlogits scaled by
        1/(B*T*grad_accum_steps), ready for ``backward``.  Returns nothing; see ``loss()``."""
        cfg, p = self.cfg, self.params
        B, T = tokens.shape
        if T > cfg.max_seq_len:
            raise ValueError("sequence length %d exceeds the model's maximum %d" % (T, cfg.max_seq_len))
        self.allocate_activations(B, T)
        a = self.acts
        L, C, NH = cfg.num_layers, cfg.channels, cfg.num_heads
        if tokens.data_ptr() != self.inputs.data_ptr():
            self.inputs.copy_(tokens, non_blocking=True)
        nvtx = self.device.type == "cuda"
        ps = self.param_sync
        if ps is not None:
            ps.wait(-1)
        ops.encoder_forward(a["encoded"], self.inputs, p["wte"], p["wpe"])
        ops.layernorm_forward(a["ln1"][0], a["ln1_mean"][0], a["ln1_rstd"][0], a["encoded"], p["ln1w"][0], p["ln1b"][0])
        for l in range(L):
          with _Range("forward layer %d" % l, nvtx):
            lln = 0 if self.recompute >= 2 else l
            lg = 0 if self.recompute >= 1 else l
            residual = a["encoded"] if l == 0 else a["residual3"][l - 1]
            ops.matmul_forward(a["qkv"][l], a["ln1"][lln], p["qkvw"][l], p["qkvb"][l], ready=(ps.flags(l) if ps is not None else None))
            ops.attention_forward(a["atty"][l], a["lse"][l], a["qkv"][l], B, T, NH)
            ops.matmul_forward(a["scratch_btc"], a["atty"][l], p["attprojw"][l], p["attprojb"][l])
            ops.fused_residual_forward(a["residual2"][l], a["ln2"][lln], a["ln2_mean"][l], a["ln2_rstd"][l], residual,
                                       a["scratch_btc"], p["ln2w"][l], p["ln2b"][l])
            ops.matmul_forward(a["fch_gelu"][lg], a["ln2"][lln], p["fcw"][l], p["fcb"][l], pre_gelu=a["fch"][l])
            ops.matmul_forward(a["scratch_btc"], a["fch_gelu"][lg], p["fcprojw"][l], p["fcprojb"][l])
            if l + 1 < L:
                nl = 0 if self.recompute >= 2 else l + 1
                ops.fused_residual_forward(a["residual3"][l], a["ln1"][nl], a["ln1_mean"][l + 1], a["ln1_rstd"][l + 1],
                                           a["residual2"][l], a["scratch_btc"], p["ln1w"][l + 1], p["ln1b"][l + 1])
            else:
                ops.fused_residual_forward(a["residual3"][l], a["lnf"], a["lnf_mean"], a["lnf_rstd"], a["residual2"][l],
                                           a["scratch_btc"], p["lnfw"], p["lnfb"])
        ops.matmul_forward(a["logits"], a["lnf"], p["wte"], None)
        if targets is not None:
            if targets.data_ptr() != self.targets.data_ptr():
                self.targets.copy_(targets, non_blocking=True)
            dloss = 1.0 / (B * T * grad_accum_steps)
            ops.fused_classifier(a["logits"], a["losses"], self.targets.view(-1), dloss, cfg.vocab_size,
                                 write_dlogits=write_dlogits, accumulate_loss=(micro_step > 0))

    def loss(self, grad_accum_steps=1):
        """Mean loss over the micro-steps accumulated so far, as a device scalar tensor (no synchronisation)."""
        B, T = self.act_shape
        out = torch.empty(1, dtype=torch.float32, device=self.device)
        ops.sum_scaled(out, self.acts["losses"], 1.0 / float(B * T * grad_accum_steps))
        return out[0]

    def logits(self):
        B, T = self.act_shape
        return self.acts["logits"].view(B, T, self.cfg.padded_vocab_size)

    # ------------------------------------------------------------------ backward
    def backward(self, micro_step=0, last_micro_step=True):
        """Backward pass of the last ``forward(tokens, targets)``.  Gradients are overwritten when micro_step == 0
        and added to otherwise.  On the last micro-step ``grad_hook(l)`` fires as soon as layer l's gradients are
        final (the ZeRO / data-parallel layer starts its reduction there, overlapping the rest of backward)."""
        cfg, p = self.cfg, self.params
        self.allocate_grads()
        g, a = self.grads, self.acts
        B, T = self.act_shape
        L, C, NH = cfg.num_layers, cfg.channels, cfg.num_heads
        acc = micro_step > 0
        hook = self.grad_hook if last_micro_step else None
        dres, dl_btc, dl_bt4c, dqkv = a["dresidual"], a["scratch_btc"], a["scratch_bt4c"], a["dqkv"]
        dlogits = a["logits"]

        ops.matmul_dgrad(dl_btc, dlogits, p["wte"])
        ops.matmul_wgrad(g["wte"], dlogits, a["lnf"], accumulate=acc)
        # every LayerNorm backward also emits the column sums of the residual-stream gradient it leaves behind: that is the
        # bias gradient of the projection (fcproj / attproj) whose output was added to the stream just before that LayerNorm
        ops.layernorm_backward(dres, g["lnfw"], g["lnfb"], dl_btc, a["residual3"][L - 1], p["lnfw"], a["lnf_mean"], a["lnf_rstd"],
                               accumulate_dinp=False, accumulate_dwdb=acc, dcolsum=g["fcprojb"][L - 1], accumulate_dcol=acc)
        nvtx = self.device.type == "cuda"
        for l in reversed(range(L)):
          with _Range("backward layer %d" % l, nvtx):
            residual = a["encoded"] if l == 0 else a["residual3"][l - 1]
            lln = 0 if self.recompute >= 2 else l
            lg = 0 if self.recompute >= 1 else l
            if self.recompute >= 1:
                ops.gelu_forward(a["fch_gelu"][lg], a["fch"][l])
            ops.matmul_dgrad(dl_bt4c, dres, p["fcprojw"][l], pre_gelu=a["fch"][l])
            ops.matmul_wgrad(g["fcprojw"][l], dres, a["fch_gelu"][lg], accumulate=acc)
            if self.recompute >= 2:
                ops.layernorm_forward(a["ln2"][lln], None, None, a["residual2"][l], p["ln2w"][l], p["ln2b"][l])
            ops.bias_grad(g["fcb"][l], dl_bt4c, accumulate=acc)
            ops.matmul_dgrad(dl_btc, dl_bt4c, p["fcw"][l])
            ops.matmul_wgrad(g["fcw"][l], dl_bt4c, a["ln2"][lln], accumulate=acc)
            ops.layernorm_backward(dres, g["ln2w"][l], g["ln2b"][l], dl_btc, a["residual2"][l], p["ln2w"][l], a["ln2_mean"][l],
                                   a["ln2_rstd"][l], accumulate_dinp=True, accumulate_dwdb=acc, dcolsum=g["attprojb"][l], accumulate_dcol=acc)
            ops.matmul_dgrad(dl_btc, dres, p["attprojw"][l])
            ops.matmul_wgrad(g["attprojw"][l], dres, a["atty"][l], accumulate=acc)
            ops.attention_backward(dqkv, dl_btc, a["qkv"][l], a["atty"][l], a["lse"][l], B, T, NH)
            if self.recompute >= 2:
                ops.layernorm_forward(a["ln1"][lln], None, None, residual, p["ln1w"][l], p["ln1b"][l])
            ops.bias_grad(g["qkvb"][l], dqkv, accumulate=acc)
            ops.matmul_dgrad(dl_btc, dqkv, p["qkvw"][l])
            ops.matmul_wgrad(g["qkvw"][l], dqkv, a["ln1"][lln], accumulate=acc)
            ops.layernorm_backward(dres, g["ln1w"][l], g["ln1b"][l], dl_btc, residual, p["ln1w"][l], a["ln1_mean"][l],
                                   a["ln1_rstd"][l], accumulate_dinp=True, accumulate_dwdb=acc,
                                   dcolsum=(g["fcprojb"][l - 1] if l > 0 else None), accumulate_dcol=acc)
            if hook is not None:
                hook(l)
        ops.encoder_backward(g["wte"], g["wpe"][:T], dres.view(B, T, C), self.inputs, accumulate_wte=True, accumulate_wpe=acc,
                             seed=(micro_step * 7919 + 13) & 0x7FFFFFFF)
        if hook is not None:
            hook(-1)

    # ------------------------------------------------------------------ bookkeeping
    def flops_per_token(self, T):
        """Model FLOPs per token as the reference counts them (train_gpt2.cu:1139-1144): 6 N + 6 L C T."""
        cfg = self.cfg
        return 6 * self.num_parameters + 6 * cfg.num_layers * cfg.channels * T
