#!/usr/bin/env python
"""Text -> flat little-endian uint16 token file (the format of ``TokenizedDataset``).

    python tools/tokenize_data.py --input corpus.txt --output data/train.bin [--tokenizer NAME] [--verify]

Reads a text file (one document per line) or a JSONL file with a ``text`` field, tokenises with a
local Hugging Face tokenizer when available (falls back to the byte tokenizer), appends EOS after
each document.  ``--verify`` re-opens the file and checks size and id range."""
import argparse
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.data.dataset import verify_token_file  # noqa: E402
from kotodama_b200.serve.app import load_tokenizer  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--tokenizer", default="HuggingFaceTB/SmolLM2-135M")
    ap.add_argument("--verify", action="store_true")
    a = ap.parse_args()
    tok = load_tokenizer(a.tokenizer)
    eos = getattr(tok, "eos_token_id", None)
    vocab = getattr(tok, "vocab_size", 65536)
    if vocab > 65536:
        raise SystemExit("vocabulary does not fit uint16")
    n = 0
    os.makedirs(os.path.dirname(os.path.abspath(a.output)), exist_ok=True)
    with open(a.output, "wb") as out:
        for line in open(a.input, errors="replace"):
            line = line.rstrip("\n")
            if not line:
                continue
            if a.input.endswith(".jsonl"):
                line = json.loads(line).get("text", "")
            ids = tok.encode(line)
            if eos is not None:
                ids = list(ids) + [eos]
            np.asarray(ids, dtype="<u2").tofile(out)
            n += len(ids)
    print(f"wrote {n} tokens to {a.output} ({type(tok).__name__})")
    if a.verify:
        info = verify_token_file(a.output, vocab)
        print("verify:", info, "OK" if info["tokens"] == n and info["in_vocab"] else "MISMATCH")


if __name__ == "__main__":
    main()
