#!/usr/bin/env python
"""Tokenise text into the ``.ds`` token files that ``Nanoset`` reads (parity: reference tools/preprocess_data.py, which
drives the datatrove pipeline).

    python tools/preprocess_data.py --tokenizer-name-or-path gpt2 --output-folder data/tok jsonl --dataset data/*.jsonl --column text
    python tools/preprocess_data.py --tokenizer-name-or-path gpt2 --output-folder data/tok hf --dataset stas/openwebtext-10k

Writes ``<output>/<shard>.ds`` (tokens, 2 or 4 bytes each), ``<shard>.ds.index`` (uint64 cumulative document ends) and
``<shard>.ds.metadata`` (``tokenizer|token_size`` then the token count).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def iter_documents(args):
    if args.readers == "jsonl":
        for path in sorted(glob.glob(args.dataset)):
            with open(path) as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)[args.column]
    elif args.readers == "hf":
        from datasets import load_dataset

        for row in load_dataset(args.dataset, split=args.split):
            yield row[args.column]
    else:
        for path in sorted(glob.glob(args.dataset)):
            with open(path) as f:
                yield f.read()


def write_token_shard(path: str, docs_tokens, token_size: int, tokenizer_name: str):
    dtype = np.uint16 if token_size == 2 else np.uint32
    ends, total = [], 0
    with open(path, "wb") as f:
        for toks in docs_tokens:
            np.asarray(toks, dtype=dtype).tofile(f)
            total += len(toks)
            ends.append(total)
    np.asarray(ends, dtype=np.uint64).tofile(path + ".index")
    with open(path + ".metadata", "w") as f:
        f.write(f"{tokenizer_name}|{token_size}\n{total}\n")
    return total


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokenizer-name-or-path", required=True)
    ap.add_argument("--eos-token", default=None)
    ap.add_argument("--output-folder", required=True)
    ap.add_argument("--shard-size", type=int, default=100_000, help="documents per output file")
    sub = ap.add_subparsers(dest="readers", required=True)
    for name in ("jsonl", "hf", "text"):
        p = sub.add_parser(name)
        p.add_argument("--dataset", required=True)
        p.add_argument("--column", default="text")
        p.add_argument("--split", default="train")
    args = ap.parse_args()
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(args.tokenizer_name_or_path)
    eos = tok.convert_tokens_to_ids(args.eos_token) if args.eos_token else tok.eos_token_id
    token_size = 4 if len(tok) > np.iinfo(np.uint16).max + 1 else 2
    os.makedirs(args.output_folder, exist_ok=True)
    shard, buf, total = 0, [], 0
    for text in iter_documents(args):
        ids = tok(text, add_special_tokens=False)["input_ids"]
        if eos is not None:
            ids = ids + [eos]
        buf.append(ids)
        if len(buf) >= args.shard_size:
            total += write_token_shard(os.path.join(args.output_folder, f"{shard:05d}.ds"), buf, token_size, args.tokenizer_name_or_path)
            shard, buf = shard + 1, []
    if buf:
        total += write_token_shard(os.path.join(args.output_folder, f"{shard:05d}.ds"), buf, token_size, args.tokenizer_name_or_path)
    print(f"wrote {total} tokens in {shard + (1 if buf else 0)} file(s) to {args.output_folder}")


if __name__ == "__main__":
    main()
