"""Converts a model checkpoint of this framework (or of the reference: same format) into a Hugging Face
``GPT2LMHeadModel`` (reference: dev/eval/export_hf.py), or a LLaMA-3 model file into a ``LlamaForCausalLM``.

    python -m llmc_b200.utils.export_hf --input log/model_00010000.bin --output gpt2_export [--dtype bfloat16]

The four matmul weights are transposed (HF's Conv1D stores (in, out)), the vocabulary padding is dropped and the
token embedding is tied to the LM head."""
import argparse

import numpy as np
import torch

from . import checkpoint


def load_tensors(path):
    cfg, version = checkpoint.read_model_header(path)
    dtype = torch.bfloat16 if version == 5 else torch.float32
    from ..models import gpt2
    shapes = gpt2.param_shapes(cfg)
    out = {}
    with open(path, "rb") as f:
        f.seek(1024)
        for name, shape in shapes:
            n = int(np.prod(shape))
            t = torch.empty(n, dtype=dtype)
            checkpoint._stream_in(f, t)
            out[name] = t.view(shape).float()
    return cfg, out


def to_hf_state_dict(cfg, w):
    sd = {"transformer.wte.weight": w["wte"][:cfg.vocab_size].clone(), "transformer.wpe.weight": w["wpe"].clone(),
          "transformer.ln_f.weight": w["lnfw"].clone(), "transformer.ln_f.bias": w["lnfb"].clone()}
    sd["lm_head.weight"] = sd["transformer.wte.weight"]
    for l in range(cfg.num_layers):
        p = "transformer.h.%d." % l
        sd[p + "ln_1.weight"], sd[p + "ln_1.bias"] = w["ln1w"][l].clone(), w["ln1b"][l].clone()
        sd[p + "attn.c_attn.weight"], sd[p + "attn.c_attn.bias"] = w["qkvw"][l].t().contiguous(), w["qkvb"][l].clone()
        sd[p + "attn.c_proj.weight"], sd[p + "attn.c_proj.bias"] = w["attprojw"][l].t().contiguous(), w["attprojb"][l].clone()
        sd[p + "ln_2.weight"], sd[p + "ln_2.bias"] = w["ln2w"][l].clone(), w["ln2b"][l].clone()
        sd[p + "mlp.c_fc.weight"], sd[p + "mlp.c_fc.bias"] = w["fcw"][l].t().contiguous(), w["fcb"][l].clone()
        sd[p + "mlp.c_proj.weight"], sd[p + "mlp.c_proj.bias"] = w["fcprojw"][l].t().contiguous(), w["fcprojb"][l].clone()
    return sd


def export_llama(path, output, dtype="bfloat16"):
    """A LLaMA-3 model file of this framework -> ``LlamaForCausalLM`` (query / key rows permuted to the rotate-half convention)."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from ..models.llama3 import Llama
    from . import llama_convert
    cfg, _ = checkpoint.read_model_header(path)
    m = Llama(cfg, "cpu", torch.float32)
    checkpoint.load_model(path, m)
    kw = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.channels, intermediate_size=cfg.hidden_dim, num_hidden_layers=cfg.num_layers,
              num_attention_heads=cfg.num_heads, num_key_value_heads=cfg.num_kv_heads, max_position_embeddings=cfg.max_seq_len,
              rms_norm_eps=cfg.norm_eps, rope_theta=cfg.rope_theta, tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    if cfg.use_scaled_rope:
        kw["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192}
    model = LlamaForCausalLM(LlamaConfig(**kw))
    missing, unexpected = model.load_state_dict(llama_convert.to_hf_state_dict(m), strict=False)
    assert not [k for k in missing if "rotary" not in k], missing
    model = model.to(getattr(torch, dtype))
    model.save_pretrained(output, max_shard_size="5GB")
    return model


def export(path, output, dtype="bfloat16"):
    if checkpoint.model_family(path) == "llama3":
        return export_llama(path, output, dtype)
    from transformers import GPT2Config, GPT2LMHeadModel
    cfg, w = load_tensors(path)
    hf_cfg = GPT2Config(vocab_size=cfg.vocab_size, n_positions=cfg.max_seq_len, n_ctx=cfg.max_seq_len, n_embd=cfg.channels,
                        n_layer=cfg.num_layers, n_head=cfg.num_heads, activation_function="gelu_new")
    model = GPT2LMHeadModel(hf_cfg)
    missing, unexpected = model.load_state_dict(to_hf_state_dict(cfg, w), strict=False)
    assert not [m for m in missing if "attn.bias" not in m and "masked_bias" not in m], missing
    model = model.to(getattr(torch, dtype))
    model.save_pretrained(output, max_shard_size="5GB")
    return model


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", "-i", required=True)
    ap.add_argument("--output", "-o", required=True)
    ap.add_argument("--dtype", "-d", default="bfloat16")
    a = ap.parse_args()
    export(a.input, a.output, a.dtype)
