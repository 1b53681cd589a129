"""LLaMA-3 family decoder on flat parameter and gradient buffers.

The reference has this family only as a PyTorch module (train_llama3.py:133-322 of the reference: RMSNorm,
rotary position embedding, grouped-query attention, SwiGLU MLP, untied LM head).  Here it is a second model family
of the same engine as GPT-2: one flat parameter buffer, one flat gradient buffer, preallocated activations,
forward and backward written out by hand on ``ops`` -- on a GPU every call is one of this library's sm_100a
kernels, on the CPU the PyTorch fp32 restatement.  The model object has the interface of ``models.gpt2.GPT``, so
the trainer, the ZeRO-1 optimizer, the in-kernel NVLink backend and the checkpoint code drive it unchanged.

Layout decisions that differ from the PyTorch module:
  * The two up-projections of the MLP (c_fc and c_fc2) live in one tensor ``fc12w`` (L, 2H, C): one GEMM produces
    both branches, one dgrad GEMM and one wgrad GEMM consume them.  Checkpoint files keep the reference's order
    (all c_fc, then all c_fc2); ``utils.checkpoint`` splits and joins.
  * Grouped-query attention is expressed as "rotate + expand": one pass turns the projection output
    (N, (NH + 2 NKV) HS) into the packed (N, 3, NH, HS) tensor the flash-attention kernels read in place, applying
    the rotary embedding on the way; its backward rotates back and sums the gradients of the repeated heads.
"""
import math
from dataclasses import dataclass

import torch

from .. import ops
from .gpt2 import _Range

PARAM_NAMES = ["wte", "ln1w", "qkvw", "attprojw", "ln2w", "fc12w", "fcprojw", "lnfw", "lmhead"]
# tensors that receive weight decay: everything two-dimensional (train_llama3.py:444-456 of the reference)
DECAYED = {"wte", "qkvw", "attprojw", "fc12w", "fcprojw", "lmhead"}
LAYERED = {"ln1w", "qkvw", "attprojw", "ln2w", "fc12w", "fcprojw"}


@dataclass
class LlamaConfig:
    max_seq_len: int = 8192
    vocab_size: int = 128256
    padded_vocab_size: int = 128256
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    channels: int = 4096
    ffn_dim_multiplier: float = 1.3
    multiple_of: int = 1024
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    use_scaled_rope: bool = True
    version: str = "3.1"

    @property
    def head_size(self):
        return self.channels // self.num_heads

    @property
    def hidden_dim(self):
        """Width of the MLP (train_llama3.py:207-214 of the reference)."""
        h = int(2 * (4 * self.channels) / 3)
        if self.ffn_dim_multiplier is not None:
            h = int(self.ffn_dim_multiplier * h)
        return self.multiple_of * ((h + self.multiple_of - 1) // self.multiple_of)


def _pad128(v):
    return (v + 127) // 128 * 128


_PRESETS = {
    # name: (L, NH, NKV, C, ffn multiplier, multiple_of)
    "8B": (32, 32, 8, 4096, 1.3, 1024),
    "70B": (80, 64, 8, 8192, 1.3, 4096),
    "405B": (126, 128, 8, 16384, 1.2, 4096),
}


def config_from_descriptor(desc):
    """'llama3:8B' | 'llama3:70B' | 'llama3:405B' (LLaMA 3.1), or a free-form list of sizes for experiments and tests:
    'llama3:l=4,c=256,h=4,kv=2,t=256,v=1024,m=64,f=1.0' (layers, channels, heads, kv heads, context, vocabulary,
    multiple_of, ffn multiplier)."""
    if not desc.startswith("llama3:"):
        raise ValueError("unknown model descriptor %r" % desc)
    body = desc[len("llama3:"):]
    if body in _PRESETS:
        L, nh, nkv, c, f, m = _PRESETS[body]
        return LlamaConfig(num_layers=L, num_heads=nh, num_kv_heads=nkv, channels=c, ffn_dim_multiplier=f, multiple_of=m)
    kv = dict(item.split("=") for item in body.split(","))
    unknown = set(kv) - set("lchtvmf") - {"kv"}
    if unknown:
        raise ValueError("unknown keys %s in %r" % (sorted(unknown), desc))
    v = int(kv.get("v", 128256))
    cfg = LlamaConfig(max_seq_len=int(kv.get("t", 8192)), vocab_size=v, padded_vocab_size=_pad128(v),
                      num_layers=int(kv.get("l", 32)), num_heads=int(kv.get("h", 32)), num_kv_heads=int(kv.get("kv", 8)),
                      channels=int(kv.get("c", 4096)), ffn_dim_multiplier=float(kv.get("f", 1.3)),
                      multiple_of=int(kv.get("m", 1024)))
    if cfg.num_heads % cfg.num_kv_heads or cfg.channels % cfg.num_heads:
        raise ValueError("heads must divide channels and kv heads must divide heads in %r" % desc)
    return cfg


def param_shapes(cfg):
    L, C, Vp, H = cfg.num_layers, cfg.channels, cfg.padded_vocab_size, cfg.hidden_dim
    qkv_rows = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size
    return [("wte", (Vp, C)), ("ln1w", (L, C)), ("qkvw", (L, qkv_rows, C)), ("attprojw", (L, C, C)), ("ln2w", (L, C)),
            ("fc12w", (L, 2 * H, C)), ("fcprojw", (L, C, H)), ("lnfw", (C,)), ("lmhead", (Vp, C))]


def num_parameters(cfg):
    return sum(math.prod(s) for _, s in param_shapes(cfg))


def rope_table(cfg, length=None):
    """(length, HS/2, 2) fp32 table of (cos, sin) of position * frequency, with the LLaMA-3.1 long-context rescaling of the
    low frequencies (train_llama3.py:81-104 and :119-129 of the reference)."""
    dim = cfg.head_size
    length = cfg.max_seq_len if length is None else length
    freqs = 1.0 / (cfg.rope_theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    if cfg.use_scaled_rope:
        scale_factor, low_factor, high_factor, old_len = 8, 1, 4, 8192
        low_wavelen, high_wavelen = old_len / low_factor, old_len / high_factor
        out = []
        for f in freqs.tolist():
            wavelen = 2 * math.pi / f
            if wavelen < high_wavelen:
                out.append(f)
            elif wavelen > low_wavelen:
                out.append(f / scale_factor)
            else:
                smooth = (old_len / wavelen - low_factor) / (high_factor - low_factor)
                out.append((1 - smooth) * f / scale_factor + smooth * f)
        freqs = torch.tensor(out, dtype=torch.float32)
    ang = torch.outer(torch.arange(length, dtype=torch.float32), freqs)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()


class Llama:
    family = "llama3"
    norm_params = ("ln1w", "ln2w")      # per-layer tensors that the forward pass reads before the layer's first GEMM
    decayed = DECAYED

    def __init__(self, cfg, device="cpu", dtype=None, recompute=1, flat_allocator=None):
        """Same contract as ``models.gpt2.GPT``: ``flat_allocator(kind, numel, dtype)`` may supply the two flat buffers
        (e.g. from symmetric memory that peer GPUs can address)."""
        self.cfg = cfg
        self.device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("parameters are bf16 (sm_100a kernels) or fp32 (full-precision mode)")
        hs = cfg.head_size
        if cfg.channels % 8 or hs % 8 or cfg.hidden_dim % 8 or (self.device.type == "cuda" and dtype == torch.bfloat16 and not 64 <= hs <= 128):
            raise ValueError("channels, head size and MLP width must be multiples of 8 and (on the GPU) the head size within 64..128")
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
        self.mean_loss = None
        self.grad_hook = None
        # set by a communication backend whose all-gather may still be in flight when forward starts (parallel/p2p.py)
        self.param_sync = None
        self.freqs = rope_table(cfg).to(self.device)

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
        """Normal(0, 0.02) weights drawn layer by layer from one mt19937 stream, residual projections scaled by
        1/sqrt(2L), norm weights 1.  (The reference script only ever loads pretrained weights; this is the GPT-2 recipe of
        train_gpt2.cu:587-642 applied to the LLaMA tensors.)"""
        from ..utils import rand
        cfg = self.cfg
        rng = rand.MT19937(seed)
        resid_std = 0.02 / math.sqrt(2.0 * cfg.num_layers)

        def fill(dst, std):
            dst.copy_(rng.normal(dst.numel(), 0.0, std).view(dst.shape))

        p = self.params
        for n in ("ln1w", "ln2w", "lnfw"):
            p[n].fill_(1.0)
        p["wte"].zero_()
        p["lmhead"].zero_()
        fill(p["wte"][:cfg.vocab_size], 0.02)
        for l in range(cfg.num_layers):
            for n, std in (("qkvw", 0.02), ("attprojw", resid_std), ("fc12w", 0.02), ("fcprojw", resid_std)):
                fill(p[n][l], std)
        fill(p["lmhead"][:cfg.vocab_size], 0.02)

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
        L, C, NH, Vp, H = cfg.num_layers, cfg.channels, cfg.num_heads, cfg.padded_vocab_size, cfg.hidden_dim
        QR = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size
        N = B * T
        Lln = 1 if self.recompute >= 2 else L
        Lg = 1 if self.recompute >= 1 else L
        e = lambda *s, dtype=dt: torch.empty(*s, dtype=dtype, device=dev)
        f32 = torch.float32
        self.acts = dict(
            encoded=e(N, C), ln1=e(Lln, N, C), ln1_rstd=e(L, N, dtype=f32), qkv_raw=e(N, QR), qkv=e(L, N, 3 * C), atty=e(L, N, C),
            lse=e(L, B, NH, T, dtype=f32), residual2=e(L, N, C), ln2=e(Lln, N, C), ln2_rstd=e(L, N, dtype=f32),
            fc12=e(L, N, 2 * H), h=e(Lg, N, H), residual3=e(L, N, C), lnf=e(N, C), lnf_rstd=e(N, dtype=f32),
            losses=torch.zeros(N, dtype=f32, device=dev), logits=e(N, Vp), scratch_btc=e(N, C), dh=e(N, H), dfc12=e(N, 2 * H),
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
        """Same contract as ``GPT.forward``: with targets the per-token losses are accumulated into ``acts['losses']`` and the
        logits buffer is turned into dlogits scaled by 1/(B*T*grad_accum_steps)."""
        cfg, p = self.cfg, self.params
        B, T = tokens.shape
        if T > cfg.max_seq_len:
            raise ValueError("sequence length %d exceeds the model's maximum %d" % (T, cfg.max_seq_len))
        self.allocate_activations(B, T)
        a = self.acts
        L, NH, NKV, eps = cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.norm_eps
        if tokens.data_ptr() != self.inputs.data_ptr():
            self.inputs.copy_(tokens, non_blocking=True)
        nvtx = self.device.type == "cuda"
        ps = self.param_sync
        if ps is not None:
            ps.wait(-1)
        ops.encoder_forward(a["encoded"], self.inputs, p["wte"], None)
        ops.rmsnorm_forward(a["ln1"][0], a["ln1_rstd"][0], a["encoded"], p["ln1w"][0], eps)
        for l in range(L):
          with _Range("forward layer %d" % l, nvtx):
            lln = 0 if self.recompute >= 2 else l
            lg = 0 if self.recompute >= 1 else l
            residual = a["encoded"] if l == 0 else a["residual3"][l - 1]
            ops.matmul_forward(a["qkv_raw"], a["ln1"][lln], p["qkvw"][l], None, ready=(ps.flags(l) if ps is not None else None))
            ops.rope_forward(a["qkv"][l], a["qkv_raw"], self.freqs, T, NH, NKV)
            ops.attention_forward(a["atty"][l], a["lse"][l], a["qkv"][l], B, T, NH)
            ops.matmul_forward(a["scratch_btc"], a["atty"][l], p["attprojw"][l], None)
            ops.rmsnorm_fused_residual_forward(a["residual2"][l], a["ln2"][lln], a["ln2_rstd"][l], residual, a["scratch_btc"],
                                               p["ln2w"][l], eps)
            ops.matmul_forward(a["fc12"][l], a["ln2"][lln], p["fc12w"][l], None)
            ops.swiglu_forward(a["h"][lg], a["fc12"][l])
            ops.matmul_forward(a["scratch_btc"], a["h"][lg], p["fcprojw"][l], None)
            if l + 1 < L:
                nl = 0 if self.recompute >= 2 else l + 1
                ops.rmsnorm_fused_residual_forward(a["residual3"][l], a["ln1"][nl], a["ln1_rstd"][l + 1], a["residual2"][l],
                                                   a["scratch_btc"], p["ln1w"][l + 1], eps)
            else:
                ops.rmsnorm_fused_residual_forward(a["residual3"][l], a["lnf"], a["lnf_rstd"], a["residual2"][l], a["scratch_btc"],
                                                   p["lnfw"], eps)
        ops.matmul_forward(a["logits"], a["lnf"], p["lmhead"], None)
        if targets is not None:
            if targets.data_ptr() != self.targets.data_ptr():
                self.targets.copy_(targets, non_blocking=True)
            dloss = 1.0 / (B * T * grad_accum_steps)
            ops.fused_classifier(a["logits"], a["losses"], self.targets.view(-1), dloss, cfg.vocab_size,
                                 write_dlogits=write_dlogits, accumulate_loss=(micro_step > 0))

    def loss(self, grad_accum_steps=1):
        B, T = self.act_shape
        out = torch.empty(1, dtype=torch.float32, device=self.device)
        ops.sum_scaled(out, self.acts["losses"], 1.0 / float(B * T * grad_accum_steps))
        return out[0]

    def logits(self):
        B, T = self.act_shape
        return self.acts["logits"].view(B, T, self.cfg.padded_vocab_size)

    # ------------------------------------------------------------------ backward
    def backward(self, micro_step=0, last_micro_step=True):
        """Backward pass of the last ``forward(tokens, targets)``; same contract as ``GPT.backward``."""
        cfg, p = self.cfg, self.params
        self.allocate_grads()
        g, a = self.grads, self.acts
        B, T = self.act_shape
        L, C, NH, NKV, eps = cfg.num_layers, cfg.channels, cfg.num_heads, cfg.num_kv_heads, cfg.norm_eps
        acc = micro_step > 0
        hook = self.grad_hook if last_micro_step else None
        dres, dl_btc, dh, dfc12, dqkv, dqkv_raw = a["dresidual"], a["scratch_btc"], a["dh"], a["dfc12"], a["dqkv"], a["qkv_raw"]
        dlogits = a["logits"]

        ops.matmul_dgrad(dl_btc, dlogits, p["lmhead"])
        ops.matmul_wgrad(g["lmhead"], dlogits, a["lnf"], accumulate=acc)
        ops.rmsnorm_backward(dres, g["lnfw"], dl_btc, a["residual3"][L - 1], p["lnfw"], a["lnf_rstd"], accumulate_dinp=False,
                             accumulate_dw=acc)
        nvtx = self.device.type == "cuda"
        for l in reversed(range(L)):
          with _Range("backward layer %d" % l, nvtx):
            residual = a["encoded"] if l == 0 else a["residual3"][l - 1]
            lln = 0 if self.recompute >= 2 else l
            lg = 0 if self.recompute >= 1 else l
            if self.recompute >= 1:
                ops.swiglu_forward(a["h"][lg], a["fc12"][l])
            ops.matmul_dgrad(dh, dres, p["fcprojw"][l])
            ops.matmul_wgrad(g["fcprojw"][l], dres, a["h"][lg], accumulate=acc)
            ops.swiglu_backward(dfc12, dh, a["fc12"][l])
            if self.recompute >= 2:
                ops.rmsnorm_forward(a["ln2"][lln], None, a["residual2"][l], p["ln2w"][l], eps)
            ops.matmul_dgrad(dl_btc, dfc12, p["fc12w"][l])
            ops.matmul_wgrad(g["fc12w"][l], dfc12, a["ln2"][lln], accumulate=acc)
            ops.rmsnorm_backward(dres, g["ln2w"][l], dl_btc, a["residual2"][l], p["ln2w"][l], a["ln2_rstd"][l], accumulate_dinp=True,
                                 accumulate_dw=acc)
            ops.matmul_dgrad(dl_btc, dres, p["attprojw"][l])
            ops.matmul_wgrad(g["attprojw"][l], dres, a["atty"][l], accumulate=acc)
            ops.attention_backward(dqkv, dl_btc, a["qkv"][l], a["atty"][l], a["lse"][l], B, T, NH)
            ops.rope_backward(dqkv_raw, dqkv, self.freqs, T, NH, NKV)
            if self.recompute >= 2:
                ops.rmsnorm_forward(a["ln1"][lln], None, residual, p["ln1w"][l], eps)
            ops.matmul_dgrad(dl_btc, dqkv_raw, p["qkvw"][l])
            ops.matmul_wgrad(g["qkvw"][l], dqkv_raw, a["ln1"][lln], accumulate=acc)
            ops.rmsnorm_backward(dres, g["ln1w"][l], dl_btc, residual, p["ln1w"][l], a["ln1_rstd"][l], accumulate_dinp=True,
                                 accumulate_dw=acc)
            if hook is not None:
                hook(l)
        ops.encoder_backward(g["wte"], None, dres.view(B, T, C), self.inputs, accumulate_wte=acc, accumulate_wpe=False,
                             seed=(micro_step * 7919 + 13) & 0x7FFFFFFF)
        if hook is not None:
            hook(-1)

    # ------------------------------------------------------------------ bookkeeping
    def flops_per_token(self, T):
        """6 N + 6 L C T, the same accounting as for GPT-2 (train_gpt2.cu:1139-1144 of the reference)."""
        cfg = self.cfg
        return 6 * self.num_parameters + 6 * cfg.num_layers * cfg.channels * T
