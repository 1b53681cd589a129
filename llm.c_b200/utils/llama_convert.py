"""LLaMA-3 weights between this framework's model and the two public layouts.

The reference script reads pretrained weights from a Hugging Face ``LlamaForCausalLM`` or from Meta's ``consolidated.*.pth``
(train_llama3.py:324-442 of the reference: ``adapt_llama_state_dict_keys_hf`` / ``adapt_llama_state_dict_keys``) and writes them
into its own ``.bin`` model file.  This module does the same for this framework, in both directions:

  from_hf_state_dict(model, sd)     Hugging Face names; the query / key projection rows are permuted back from the
                                    "rotate half" convention to the interleaved (complex pair) convention the kernels use
  to_hf_state_dict(model)           the inverse (what a ``LlamaForCausalLM`` of the same sizes loads)
  from_meta_state_dict(model, sd)   Meta names (no permutation)

``python -m llmc_b200.utils.llama_convert --hf-dir <local directory> --out llama3.bin`` converts a local Hugging Face checkpoint
into a model file that ``train_llama3.py --model llama3.bin`` loads (nothing is downloaded).

Layout reminders: ``qkvw[l]`` = [wq; wk; wv] rows; ``fc12w[l]`` = [up_proj (linear branch); gate_proj (SiLU branch)] rows;
the vocabulary dimension of ``wte`` / ``lmhead`` is padded to a multiple of 128 with zero rows.
"""
import argparse
import sys

import torch


def _unpermute(w, n_heads):
    """Hugging Face (rotate-half) -> interleaved pairs, for a (n_heads * hs, C) projection."""
    d1, d2 = w.shape
    return w.view(n_heads, 2, d1 // n_heads // 2, d2).transpose(1, 2).reshape(d1, d2)


def _permute(w, n_heads):
    """Interleaved pairs -> Hugging Face (rotate-half)."""
    d1, d2 = w.shape
    return w.view(n_heads, d1 // n_heads // 2, 2, d2).transpose(1, 2).reshape(d1, d2)


def _put(dst, src):
    if tuple(dst.shape) != tuple(src.shape):
        raise ValueError("shape mismatch: model %s, checkpoint %s" % (tuple(dst.shape), tuple(src.shape)))
    dst.copy_(src)


def _load_common(model, wte, lmhead, lnf, layers):
    """layers: list of dicts(ln1, wq, wk, wv, wo, ln2, up, gate, down) already in the interleaved convention."""
    cfg, p = model.cfg, model.params
    V = cfg.vocab_size
    p["wte"].zero_()
    p["lmhead"].zero_()
    _put(p["wte"][:V], wte)
    _put(p["lmhead"][:V], lmhead)
    _put(p["lnfw"], lnf)
    H = cfg.hidden_dim
    for l, t in enumerate(layers):
        _put(p["ln1w"][l], t["ln1"])
        _put(p["qkvw"][l], torch.cat([t["wq"], t["wk"], t["wv"]], dim=0))
        _put(p["attprojw"][l], t["wo"])
        _put(p["ln2w"][l], t["ln2"])
        _put(p["fc12w"][l, :H], t["up"])
        _put(p["fc12w"][l, H:], t["gate"])
        _put(p["fcprojw"][l], t["down"])


def from_hf_state_dict(model, sd):
    cfg = model.cfg
    layers = []
    for l in range(cfg.num_layers):
        k = "model.layers.%d." % l
        layers.append(dict(ln1=sd[k + "input_layernorm.weight"], wq=_unpermute(sd[k + "self_attn.q_proj.weight"], cfg.num_heads),
                           wk=_unpermute(sd[k + "self_attn.k_proj.weight"], cfg.num_kv_heads), wv=sd[k + "self_attn.v_proj.weight"],
                           wo=sd[k + "self_attn.o_proj.weight"], ln2=sd[k + "post_attention_layernorm.weight"],
                           up=sd[k + "mlp.up_proj.weight"], gate=sd[k + "mlp.gate_proj.weight"], down=sd[k + "mlp.down_proj.weight"]))
    lmhead = sd["lm_head.weight"] if "lm_head.weight" in sd else sd["model.embed_tokens.weight"]      # tied checkpoints
    _load_common(model, sd["model.embed_tokens.weight"], lmhead, sd["model.norm.weight"], layers)


def from_meta_state_dict(model, sd):
    cfg = model.cfg
    layers = []
    for l in range(cfg.num_layers):
        k = "layers.%d." % l
        layers.append(dict(ln1=sd[k + "attention_norm.weight"], wq=sd[k + "attention.wq.weight"], wk=sd[k + "attention.wk.weight"],
                           wv=sd[k + "attention.wv.weight"], wo=sd[k + "attention.wo.weight"], ln2=sd[k + "ffn_norm.weight"],
                           up=sd[k + "feed_forward.w3.weight"], gate=sd[k + "feed_forward.w1.weight"], down=sd[k + "feed_forward.w2.weight"]))
    _load_common(model, sd["tok_embeddings.weight"], sd["output.weight"], sd["norm.weight"], layers)


def to_hf_state_dict(model):
    cfg, p = model.cfg, model.params
    V, H, hs = cfg.vocab_size, cfg.hidden_dim, cfg.head_size
    nq, nkv = cfg.num_heads * hs, cfg.num_kv_heads * hs
    f = lambda t: t.detach().float().cpu().clone()
    sd = {"model.embed_tokens.weight": f(p["wte"][:V]), "model.norm.weight": f(p["lnfw"]), "lm_head.weight": f(p["lmhead"][:V])}
    for l in range(cfg.num_layers):
        k = "model.layers.%d." % l
        qkv = f(p["qkvw"][l])
        sd[k + "input_layernorm.weight"] = f(p["ln1w"][l])
        sd[k + "self_attn.q_proj.weight"] = _permute(qkv[:nq], cfg.num_heads)
        sd[k + "self_attn.k_proj.weight"] = _permute(qkv[nq:nq + nkv], cfg.num_kv_heads)
        sd[k + "self_attn.v_proj.weight"] = qkv[nq + nkv:].clone()
        sd[k + "self_attn.o_proj.weight"] = f(p["attprojw"][l])
        sd[k + "post_attention_layernorm.weight"] = f(p["ln2w"][l])
        sd[k + "mlp.up_proj.weight"] = f(p["fc12w"][l, :H])
        sd[k + "mlp.gate_proj.weight"] = f(p["fc12w"][l, H:])
        sd[k + "mlp.down_proj.weight"] = f(p["fcprojw"][l])
    return sd


def config_from_hf(hf_cfg):
    """A LlamaConfig of this framework for a Hugging Face ``LlamaConfig`` (its MLP width must be reachable through
    ffn_dim_multiplier / multiple_of: the width is stored that way in the model file header)."""
    from ..models.llama3 import LlamaConfig, _pad128
    C, inter = hf_cfg.hidden_size, hf_cfg.intermediate_size
    base = int(2 * (4 * C) / 3)
    scaling = getattr(hf_cfg, "rope_scaling", None) or getattr(hf_cfg, "rope_parameters", None) or {}
    scaled = isinstance(scaling, dict) and (scaling.get("rope_type") == "llama3" or scaling.get("type") == "llama3")
    theta = getattr(hf_cfg, "rope_theta", None)
    if theta is None and isinstance(scaling, dict):
        theta = scaling.get("rope_theta")
    for mult_of in (inter, 4096, 1024, 256, 128, 64, 32, 16, 8):
        if inter % mult_of:
            continue
        cfg = LlamaConfig(max_seq_len=hf_cfg.max_position_embeddings, vocab_size=hf_cfg.vocab_size, padded_vocab_size=_pad128(hf_cfg.vocab_size),
                          num_layers=hf_cfg.num_hidden_layers, num_heads=hf_cfg.num_attention_heads, num_kv_heads=hf_cfg.num_key_value_heads,
                          channels=C, ffn_dim_multiplier=inter / base, multiple_of=mult_of, norm_eps=hf_cfg.rms_norm_eps,
                          rope_theta=float(theta if theta is not None else 500000.0), use_scaled_rope=bool(scaled))
        if cfg.hidden_dim == inter:
            return cfg
    raise ValueError("cannot express an MLP width of %d for %d channels" % (inter, C))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hf-dir", required=True, help="local directory of a Hugging Face LLaMA-3 checkpoint")
    ap.add_argument("--out", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    a = ap.parse_args(argv)
    from transformers import AutoModelForCausalLM
    from ..models.llama3 import Llama
    from . import checkpoint
    hf = AutoModelForCausalLM.from_pretrained(a.hf_dir, local_files_only=True)
    model = Llama(config_from_hf(hf.config), "cpu", torch.bfloat16 if a.dtype == "bfloat16" else torch.float32)
    from_hf_state_dict(model, hf.state_dict())
    checkpoint.write_model(a.out, model)
    print("wrote %s (%d parameters)" % (a.out, model.num_parameters))
    return 0


if __name__ == "__main__":
    sys.exit(main())
