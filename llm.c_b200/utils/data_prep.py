"""Dataset preparation helpers (reference: dev/data/*.py).  The reference's scripts download text from the Hub and
tokenize it with tiktoken; neither a network nor tiktoken is assumed here, so these helpers take any ``encode``
callable (text -> list of token ids) and write the same shard / evaluation files:

  shard_documents()   documents -> <prefix>_val_000000.bin (first shard) + <prefix>_train_%06d.bin, each document prefixed
                      by the end-of-text token, ``shard_size`` tokens per shard (reference: dev/data/fineweb.py:96-143)
  write_split()       one tokenized stream -> <prefix>_val.bin (first ``val_tokens``) + <prefix>_train.bin
                      (reference: dev/data/tinyshakespeare.py)
  render_hellaswag()  HellaSwag jsonl -> examples for ``write_evalfile`` (reference: dev/data/hellaswag.py)
  render_mmlu()       MMLU rows -> the same multiple-choice format (reference: dev/data/mmlu.py)
"""
import json

import numpy as np

from .dataloader import write_datafile, write_evalfile


def shard_documents(docs, encode, prefix, eot=50256, shard_size=10 ** 8, model_desc="gpt-2"):
    """docs: iterable of strings.  Returns the list of files written.  ``model_desc`` "llama-3" writes uint32 shards
    (pass that tokenizer's end-of-text id, 128000 in the reference, as ``eot``)."""
    wide = model_desc == "llama-3"
    files, buf, count, shard = [], np.empty(shard_size, dtype=np.uint32 if wide else np.uint16), 0, 0

    def flush(n):
        nonlocal shard
        split = "val" if shard == 0 else "train"
        path = "%s_%s_%06d.bin" % (prefix, split, shard)
        write_datafile(path, buf[:n], model_desc)
        files.append(path)
        shard += 1

    for doc in docs:
        toks = np.asarray([eot] + list(encode(doc)), dtype=np.int64)
        if not wide and toks.max(initial=0) >= 2 ** 16:
            raise ValueError("token id does not fit uint16")
        toks = toks.astype(buf.dtype)
        while toks.size:
            take = min(shard_size - count, toks.size)
            buf[count:count + take] = toks[:take]
            count += take
            toks = toks[take:]
            if count == shard_size:
                flush(count)
                count = 0
    if count:
        flush(count)
    return files


def write_split(tokens, prefix, val_tokens=32768, model_desc="gpt-2"):
    tokens = np.asarray(tokens, dtype=np.uint32 if model_desc == "llama-3" else np.uint16)
    write_datafile(prefix + "_val.bin", tokens[:val_tokens], model_desc)
    write_datafile(prefix + "_train.bin", tokens[val_tokens:], model_desc)
    return prefix + "_train.bin", prefix + "_val.bin"


def render_hellaswag(jsonl_path, encode):
    """One example per line of the HellaSwag jsonl: context tokens, four endings (encoded with a leading space), label."""
    examples = []
    with open(jsonl_path) as f:
        for line in f:
            ex = json.loads(line)
            examples.append(dict(ctx=list(encode(ex["ctx"])), endings=[list(encode(" " + e)) for e in ex["endings"]], label=int(ex["label"])))
    return examples


def render_mmlu(rows, encode):
    """rows: dicts(question, choices[4], answer index).  Completion-style rendering as in the reference."""
    examples = []
    for r in rows:
        ctx = "Question: %s\n\nAnswer:" % r["question"]
        examples.append(dict(ctx=list(encode(ctx)), endings=[list(encode(" " + c)) for c in r["choices"]], label=int(r["answer"])))
    return examples


def write_eval(path, examples):
    write_evalfile(path, examples)
