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


# ---------------------------------------------------------------------------------------------------------------
# per-dataset entry points (reference: dev/data/{tinyshakespeare,tinystories,fineweb,hellaswag,mmlu}.py).  The reference's
# scripts download their input; here the input is a local file that the user has fetched, so the scripts run offline.

def get_encoder(name):
    """'gpt2' -> tiktoken's GPT-2 encoding (must be installed with its vocabulary cached); 'bytes' -> one token per UTF-8 byte
    (for smoke tests: ids 0..255, end of text 256)."""
    if name == "bytes":
        return (lambda s: list(s.encode("utf-8"))), 256
    if name == "gpt2":
        try:
            import tiktoken
        except ImportError as e:
            raise SystemExit("the gpt2 encoder needs the tiktoken package (and its cached vocabulary): %s" % e)
        enc = tiktoken.get_encoding("gpt2")
        return (lambda s: enc.encode_ordinary(s)), enc._special_tokens["<|endoftext|>"]
    raise SystemExit("unknown encoder %r (gpt2 | bytes)" % name)


def prepare_tinyshakespeare(text_path, out_prefix, encode, eot, val_tokens=32768):
    """One text file; blank-line separated sections each start with the end-of-text token; the first ``val_tokens`` tokens are
    the validation split (reference: dev/data/tinyshakespeare.py:40-66)."""
    with open(text_path) as f:
        text = f.read()
    toks = []
    for section in text.split("\n\n"):
        toks.append(eot)
        toks.extend(encode(section + "\n\n"))
    return write_split(toks, out_prefix, val_tokens)


def prepare_tinystories(json_paths, out_prefix, encode, eot, shard_size=10 ** 8):
    """TinyStories json shards (lists of {"story": ...}); first shard of the output is the validation split."""
    def docs():
        for p in json_paths:
            with open(p) as f:
                for ex in json.load(f):
                    yield ex["story"].strip()
    return shard_documents(docs(), encode, out_prefix, eot, shard_size)


def prepare_fineweb(jsonl_paths, out_prefix, encode, eot, shard_size=10 ** 8):
    """FineWeb / FineWeb-EDU as jsonl with a "text" field per line -> 100 M-token shards, shard 0 = validation
    (reference: dev/data/fineweb.py:96-143)."""
    def docs():
        for p in jsonl_paths:
            with open(p) as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)["text"]
    return shard_documents(docs(), encode, out_prefix, eot, shard_size)


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="tokenize a local copy of one of the reference's datasets into .bin files")
    ap.add_argument("dataset", choices=["tinyshakespeare", "tinystories", "fineweb", "hellaswag", "mmlu"])
    ap.add_argument("inputs", nargs="+", help="local input file(s): text, json shards, jsonl, HellaSwag jsonl, MMLU json rows")
    ap.add_argument("-o", "--out", required=True, help="output prefix (train/val shards) or output file (eval sets)")
    ap.add_argument("--encoder", default="gpt2")
    ap.add_argument("--shard-size", type=int, default=10 ** 8)
    a = ap.parse_args(argv)
    encode, eot = get_encoder(a.encoder)
    if a.dataset == "tinyshakespeare":
        files = prepare_tinyshakespeare(a.inputs[0], a.out, encode, eot)
    elif a.dataset == "tinystories":
        files = prepare_tinystories(a.inputs, a.out, encode, eot, a.shard_size)
    elif a.dataset == "fineweb":
        files = prepare_fineweb(a.inputs, a.out, encode, eot, a.shard_size)
    elif a.dataset == "hellaswag":
        write_eval(a.out, render_hellaswag(a.inputs[0], encode))
        files = [a.out]
    else:
        with open(a.inputs[0]) as f:
            write_eval(a.out, render_mmlu(json.load(f), encode))
        files = [a.out]
    for p in files:
        print("wrote %s" % p)
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
