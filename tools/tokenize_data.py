#!/usr/bin/env python
"""Text -> flat little-endian uint16 token file (the format ``TokenizedDataset`` memory-maps).

    python tools/tokenize_data.py --input corpus.txt --output data/train.bin
    python tools/tokenize_data.py --dataset HuggingFaceFW/fineweb-edu --name sample-10BT --output data/fw.bin \\
        --max_tokens 2000000000
    python tools/tokenize_data.py --verify data/train.bin

Sources: a local text file (one document per line), a JSONL file (``--text_field``), or a Hugging
Face dataset that is already in the local cache (``--dataset/--name/--split``, streamed in batches
of ``--batch_size`` documents; there is no network here, so nothing is downloaded).  Documents are
tokenised in batches with a local Hugging Face tokenizer when one is available (the byte tokenizer
otherwise), EOS is appended after each document, and ids are written as uint16 (the vocabulary
must fit).  ``--verify`` re-opens a file and reports size, id range and the first tokens, as the
reference's tool does (``scripts/utils/tokenize_data.py:164-176``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Iterable, Iterator, Optional

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.data.dataset import verify_token_file  # noqa: E402
from kotodama_b200.data.tokenizer import load_tokenizer  # noqa: E402


def iter_documents(a: argparse.Namespace) -> Iterator[str]:
    if a.dataset:
        try:
            from datasets import load_dataset
        except ImportError as e:                    # pragma: no cover - optional dependency
            raise SystemExit(f"--dataset needs the 'datasets' package: {e}")
        ds = load_dataset(a.dataset, a.name, split=a.split, streaming=True)
        for row in ds:
            yield row.get(a.text_field, "") or ""
        return
    with open(a.input, errors="replace") as fh:
        jsonl = a.input.endswith(".jsonl") or a.input.endswith(".json")
        for line in fh:
            line = line.rstrip("\n")
            if not line:
                continue
            yield (json.loads(line).get(a.text_field, "") or "") if jsonl else line


def batches(it: Iterable[str], n: int) -> Iterator[list[str]]:
    cur: list[str] = []
    for x in it:
        cur.append(x)
        if len(cur) >= n:
            yield cur
            cur = []
    if cur:
        yield cur


def encode_batch(tok, docs: list[str]) -> list[list[int]]:
    """Batched encoding when the tokenizer offers it (Hugging Face fast tokenizers), else one by one."""
    if hasattr(tok, "__call__") and hasattr(tok, "batch_encode_plus"):
        return tok(docs, add_special_tokens=False)["input_ids"]
    return [list(tok.encode(d)) for d in docs]


def tokenize(a: argparse.Namespace) -> int:
    tok = load_tokenizer(a.tokenizer)
    eos: Optional[int] = getattr(tok, "eos_token_id", None)
    vocab = int(getattr(tok, "vocab_size", 65536))
    if len(tok) > 65536 if hasattr(tok, "__len__") else vocab > 65536:
        raise SystemExit("vocabulary does not fit uint16")
    os.makedirs(os.path.dirname(os.path.abspath(a.output)), exist_ok=True)
    tmp = a.output + ".tmp"
    n_tok = n_doc = 0
    t0 = last = time.time()
    with open(tmp, "wb") as out:
        for docs in batches(iter_documents(a), a.batch_size):
            for ids in encode_batch(tok, docs):
                ids = list(ids) + ([eos] if eos is not None else [])
                if a.max_tokens is not None and n_tok + len(ids) > a.max_tokens:
                    ids = ids[: max(0, a.max_tokens - n_tok)]
                np.asarray(ids, dtype="<u2").tofile(out)
                n_tok += len(ids)
                n_doc += 1
                if a.max_tokens is not None and n_tok >= a.max_tokens:
                    break
            if time.time() - last > 10:
                last = time.time()
                print(f"  {n_doc:,} documents, {n_tok:,} tokens, {n_tok / max(last - t0, 1e-9) / 1e6:.2f} M tok/s", flush=True)
            if a.max_tokens is not None and n_tok >= a.max_tokens:
                break
    os.replace(tmp, a.output)                       # a partial file never carries the final name
    dt = time.time() - t0
    print(f"wrote {n_tok:,} tokens from {n_doc:,} documents to {a.output} "
          f"({os.path.getsize(a.output) / 1e6:.1f} MB, {type(tok).__name__}, {dt:.1f} s)")
    info = verify_token_file(a.output, vocab)
    print("verify:", info, "OK" if info["tokens"] == n_tok and info["in_vocab"] else "MISMATCH")
    return n_tok


def verify(path: str, vocab: Optional[int]) -> None:
    info = verify_token_file(path, vocab or 65536)
    arr = np.memmap(path, dtype="<u2", mode="r")
    print(f"{path}: {info['tokens']:,} tokens, {os.path.getsize(path) / 1e6:.1f} MB, id range [{int(arr.min())}, {int(arr.max())}]"
          f", in vocabulary: {info['in_vocab']}")
    print("first 16 ids:", arr[:16].tolist())
    counts = np.bincount(np.asarray(arr[: min(len(arr), 5_000_000)]), minlength=1)
    top = np.argsort(counts)[::-1][:5]
    print("most frequent ids in the first 5 M tokens:", [(int(i), int(counts[i])) for i in top])


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", help="text or JSONL file")
    ap.add_argument("--dataset", help="Hugging Face dataset name (local cache)")
    ap.add_argument("--name", default=None, help="dataset config name")
    ap.add_argument("--split", default="train")
    ap.add_argument("--text_field", default="text")
    ap.add_argument("--tokenizer", default="HuggingFaceTB/SmolLM2-135M")
    ap.add_argument("--output", help="output .bin path")
    ap.add_argument("--max_tokens", type=int, default=None)
    ap.add_argument("--batch_size", type=int, default=1000, help="documents per tokenizer call")
    ap.add_argument("--vocab_size", type=int, default=None, help="for --verify: ids must stay below this")
    ap.add_argument("--verify", nargs="?", const="", default=None,
                    help="with a path: only verify that file; without: verify the output after writing (always done)")
    a = ap.parse_args()
    if a.verify:
        verify(a.verify, a.vocab_size)
        return
    if not a.output or not (a.input or a.dataset):
        ap.error("--output and one of --input / --dataset are required")
    tokenize(a)


if __name__ == "__main__":
    main()
