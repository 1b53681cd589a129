"""Autograd oracle: the GPT-2 forward pass written with ordinary differentiable PyTorch ops on fp32 copies of a
model's parameters (the role train_gpt2.py plays for the reference's tests)."""
import math

import torch
import torch.nn.functional as F


def oracle_loss_and_grads(model, tokens, targets):
    cfg = model.cfg
    p = {k: v.detach().float().cpu().clone().requires_grad_(True) for k, v in model.params.items()}
    B, T = tokens.shape
    C, NH = cfg.channels, cfg.num_heads
    x = p["wte"][tokens.long()] + p["wpe"][:T]
    for l in range(cfg.num_layers):
        h = F.layer_norm(x, (C,), p["ln1w"][l], p["ln1b"][l], 1e-5)
        qkv = h @ p["qkvw"][l].t() + p["qkvb"][l]
        q, k, v = qkv.view(B, T, 3, NH, C // NH).unbind(2)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        att = (q @ k.transpose(-1, -2)) / math.sqrt(C // NH)
        att = att.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
        y = (torch.softmax(att, -1) @ v).transpose(1, 2).reshape(B, T, C)
        x = x + y @ p["attprojw"][l].t() + p["attprojb"][l]
        h = F.layer_norm(x, (C,), p["ln2w"][l], p["ln2b"][l], 1e-5)
        h = F.gelu(h @ p["fcw"][l].t() + p["fcb"][l], approximate="tanh")
        x = x + h @ p["fcprojw"][l].t() + p["fcprojb"][l]
    x = F.layer_norm(x, (C,), p["lnfw"], p["lnfb"], 1e-5)
    logits = x @ p["wte"].t()
    loss = F.cross_entropy(logits[..., :cfg.vocab_size].reshape(B * T, -1), targets.reshape(-1).long())
    loss.backward()
    return logits.detach(), loss.item(), {k: v.grad for k, v in p.items()}


def llama_oracle_loss_and_grads(model, tokens, targets):
    """The LLaMA-3 forward pass with differentiable PyTorch ops: complex-number rotary embedding, repeat_interleave for the
    grouped-query heads, silu-gated MLP (the role train_llama3.py plays in the reference)."""
    cfg = model.cfg
    p = {k: v.detach().float().cpu().clone().requires_grad_(True) for k, v in model.params.items()}
    B, T = tokens.shape
    C, NH, NKV, HS, H = cfg.channels, cfg.num_heads, cfg.num_kv_heads, cfg.head_size, cfg.hidden_dim
    tab = model.freqs.detach().float().cpu()[:T]
    rot = torch.complex(tab[..., 0], tab[..., 1]).view(1, T, 1, HS // 2)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w

    def rope(t):
        tc = torch.view_as_complex(t.reshape(*t.shape[:-1], -1, 2).contiguous())
        return torch.view_as_real(tc * rot).flatten(3)

    x = p["wte"][tokens.long()]
    for l in range(cfg.num_layers):
        qkv = rms(x, p["ln1w"][l]) @ p["qkvw"][l].t()
        q, k, v = qkv.split([NH * HS, NKV * HS, NKV * HS], dim=-1)
        q, k, v = q.view(B, T, NH, HS), k.view(B, T, NKV, HS), v.view(B, T, NKV, HS)
        q, k = rope(q), rope(k)
        k, v = k.repeat_interleave(NH // NKV, dim=2), v.repeat_interleave(NH // NKV, dim=2)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
        x = x + y @ p["attprojw"][l].t()
        h = rms(x, p["ln2w"][l]) @ p["fc12w"][l].t()
        x = x + (h[..., :H] * F.silu(h[..., H:])) @ p["fcprojw"][l].t()
    logits = rms(x, p["lnfw"]) @ p["lmhead"].t()
    loss = F.cross_entropy(logits[..., :cfg.vocab_size].reshape(B * T, -1), targets.reshape(-1).long())
    loss.backward()
    return logits.detach(), loss.item(), {k: v.grad for k, v in p.items()}
