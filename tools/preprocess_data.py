"""Tokenise a text dataset into flat ``uint16`` token files (``train.bin``, ``validation.bin``).

Same CLI and output format as the reference tool (tools/preprocess_data.py:57-66): Hugging
Face ``datasets`` + a GPT-2 fast tokenizer, empty lines dropped, lines tokenised in batches
of 1000 without special tokens, an EOS token appended to every line, ids written with
``ndarray.tofile``. Needs network or a warm HF cache; ``--text-file`` tokenises a local text
file instead, and ``tools/make_synthetic_data.py`` makes random token files offline.
"""
from __future__ import annotations

import argparse
import os

import numpy as np


def _encode_lines(lines, tokenizer, batch_size=1000):
    eos = tokenizer.eos_token_id
    ids: list[int] = []
    for i in range(0, len(lines), batch_size):
        enc = tokenizer(lines[i:i + batch_size], add_special_tokens=False)["input_ids"]
        for seq in enc:
            ids.extend(seq)
            ids.append(eos)
    return np.asarray(ids, dtype=np.uint16)


def preprocess_wikitext(args):
    from transformers import GPT2TokenizerFast
    tokenizer = GPT2TokenizerFast.from_pretrained(args.tokenizer_name)
    os.makedirs(args.output_dir, exist_ok=True)
    if args.text_file:
        with open(args.text_file, encoding="utf-8") as f:
            splits = {"train": [ln for ln in f.read().splitlines() if ln.strip()]}
    else:
        from datasets import load_dataset
        ds = load_dataset(args.dataset_name, args.dataset_config_name)
        splits = {name: [t for t in ds[name]["text"] if t.strip()] for name in ("train", "validation") if name in ds}
    for name, lines in splits.items():
        arr = _encode_lines(lines, tokenizer)
        out = os.path.join(args.output_dir, f"{name}.bin")
        arr.tofile(out)
        print(f"{name}: {len(lines)} lines -> {arr.size} tokens -> {out}")


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("--dataset_name", type=str, default="wikitext")
    p.add_argument("--dataset_config_name", type=str, default="wikitext-103-v1")
    p.add_argument("--tokenizer_name", type=str, default="gpt2")
    p.add_argument("--output_dir", type=str, default="data/wikitext_bin")
    p.add_argument("--text-file", type=str, default=None, help="tokenise this local file instead of a HF dataset")
    preprocess_wikitext(p.parse_args())
