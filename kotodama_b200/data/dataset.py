"""Token datasets.

The reference's training loop imports ``RandomTokenDataset`` and ``TokenizedDataset`` from a
module that is absent from its repository (``src/training/train.py:47``, usage at
``train.py:420-449`` and ``:475-477``); the on-disk format is documented by its tokenizer tool:
a flat little-endian uint16 token file (``scripts/utils/tokenize_data.py:156-159``).  Both
classes are infinite iterables yielding ``LongTensor[seq_len]`` and are resumable through
``state_dict`` / ``load_state_dict``.
"""
from __future__ import annotations

from typing import Any, Iterator

import numpy as np
import torch
from torch.utils.data import IterableDataset


class RandomTokenDataset(IterableDataset):
    """Uniform-random token ids in ``[0, vocab_size)``; stream ``k`` of rank ``r`` is a pure
    function of ``(seed, r, k)`` so a resumed run continues the same stream."""

    def __init__(self, vocab_size: int, seq_len: int, seed: int = 42, rank: int = 0, fixed: bool = False) -> None:
        self.vocab_size, self.seq_len, self.seed, self.rank = vocab_size, seq_len, seed, rank
        self.fixed = fixed          # repeat a small fixed set of sequences (learnability checks)
        self.position = 0

    def _sample(self, index: int) -> torch.Tensor:
        g = torch.Generator().manual_seed((self.seed * 1_000_003 + self.rank) * 1_000_003 + index)
        return torch.randint(0, self.vocab_size, (self.seq_len,), generator=g, dtype=torch.long)

    def __iter__(self) -> Iterator[torch.Tensor]:
        while True:
            idx = self.position % 8 if self.fixed else self.position
            self.position += 1
            yield self._sample(idx)

    def state_dict(self) -> dict[str, Any]:
        return {"position": self.position, "seed": self.seed, "rank": self.rank}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.position = int(state.get("position", 0))


class TokenizedDataset(IterableDataset):
    """Flat uint16 token file cut into ``seq_len`` windows.

    Windows are visited in a seeded permutation per epoch; rank ``r`` of ``world_size`` takes
    windows ``r, r+world_size, ...`` of that permutation, so ranks never overlap within an epoch.
    """

    def __init__(self, path: str, seq_len: int, rank: int = 0, world_size: int = 1, seed: int = 42) -> None:
        self.path, self.seq_len, self.rank, self.world_size, self.seed = path, seq_len, rank, world_size, seed
        self.tokens = np.memmap(path, dtype=np.uint16, mode="r")
        self.n_windows = len(self.tokens) // seq_len
        if self.n_windows < world_size:
            raise ValueError(f"{path}: {len(self.tokens)} tokens give {self.n_windows} windows of {seq_len}, "
                             f"fewer than world_size={world_size}")
        self.epoch = 0
        self.index = 0              # position inside this rank's slice of the epoch permutation

    def _perm(self, epoch: int) -> np.ndarray:
        return np.random.default_rng(self.seed + 7919 * epoch).permutation(self.n_windows)[self.rank::self.world_size]

    def __iter__(self) -> Iterator[torch.Tensor]:
        while True:
            perm = self._perm(self.epoch)
            while self.index < len(perm):
                w = int(perm[self.index])
                self.index += 1
                arr = np.asarray(self.tokens[w * self.seq_len:(w + 1) * self.seq_len]).astype(np.int64)
                yield torch.from_numpy(arr)
            self.epoch += 1
            self.index = 0

    def state_dict(self) -> dict[str, Any]:
        return {"epoch": self.epoch, "index": self.index, "seed": self.seed}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.epoch = int(state.get("epoch", 0))
        self.index = int(state.get("index", 0))


def write_token_file(path: str, tokens: Any) -> None:
    """Write tokens in the flat uint16 format (vocabularies up to 65 535)."""
    arr = np.asarray(tokens)
    if arr.size and (arr.min() < 0 or arr.max() > 65535):
        raise ValueError("token ids must fit uint16")
    arr.astype("<u2").tofile(path)


def verify_token_file(path: str, vocab_size: int) -> dict[str, Any]:
    """The tokenizer tool's ``--verify``: size, id range and a histogram head."""
    arr = np.memmap(path, dtype=np.uint16, mode="r")
    return {"tokens": int(arr.size), "min": int(arr.min()) if arr.size else 0,
            "max": int(arr.max()) if arr.size else 0, "in_vocab": bool(arr.size == 0 or arr.max() < vocab_size)}


class BatchIterator:
    """Stacks ``micro_batch`` sequences into pinned ``LongTensor[mb, seq]`` batches."""

    def __init__(self, dataset: IterableDataset, micro_batch: int, pin: bool = False) -> None:
        self.dataset, self.micro_batch, self.pin = dataset, micro_batch, pin
        self._it = iter(dataset)

    def __iter__(self) -> "BatchIterator":
        return self

    def __next__(self) -> torch.Tensor:
        rows = []
        for _ in range(self.micro_batch):
            try:
                rows.append(next(self._it))
            except StopIteration:       # finite dataset: restart (``train.py:592-597``)
                self._it = iter(self.dataset)
                rows.append(next(self._it))
        b = torch.stack(rows)
        return b.pin_memory() if self.pin and torch.cuda.is_available() else b
