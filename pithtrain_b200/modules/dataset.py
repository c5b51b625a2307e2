"""Token datasets: memory-mapped ``.bin`` shards with a global shuffle, and a synthetic stream.

A ``.bin`` file is what the tokenizer task writes: ``np.save`` of the token array (followed by a
second array of document split points, ignored here). Only touched pages are read. ``ConcatDataset``
writes ``offsets.npy`` / ``indices.npy`` once per node (local rank 0) and every rank memory-maps
them after a barrier — the contract of pithtrain/modules/dataset.py:19-93. ``SyntheticDataset``
produces uniform token ids from a counter-based generator so benchmarks need no files.
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import List, Tuple

import numpy as np
import torch
import torch.distributed as dist


class MemmapDataset:
    def __init__(self, path: Path, sequence_length: int):
        self.root = Path(path).parent
        self.sequence_length = sequence_length
        self.tokens = np.load(path, mmap_mode="r")

    def __len__(self) -> int:
        return max(0, (len(self.tokens) - 1) // self.sequence_length)

    def __getitem__(self, idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.get_chunk(idx, 0, self.sequence_length)

    def get_chunk(self, idx: int, seq_offset: int, seq_length: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Tokens ``[seq_offset, seq_offset+seq_length)`` of sequence ``idx`` and their next-token labels."""
        start = int(idx) * self.sequence_length + seq_offset
        window = np.asarray(self.tokens[start:start + seq_length + 1]).astype(np.int64)
        return torch.from_numpy(window[:-1].copy()), torch.from_numpy(window[1:].copy())


class ConcatDataset:
    OFFSETS = "offsets.npy"
    INDICES = "indices.npy"

    def __init__(self, memmap_datasets: List[MemmapDataset], seed: int):
        assert memmap_datasets, "no *.bin files found in the dataset directory"
        self.memmap_datasets = memmap_datasets
        root = os.path.commonpath([str(d.root) for d in memmap_datasets])
        offsets_path, indices_path = Path(root, self.OFFSETS), Path(root, self.INDICES)
        if int(os.environ.get("LOCAL_RANK", "0")) == 0:
            offsets = np.cumsum([len(ds) for ds in memmap_datasets])
            np.save(offsets_path, offsets)
            gen = torch.Generator().manual_seed(seed)
            np.save(indices_path, torch.randperm(int(offsets[-1]), generator=gen).numpy())
        if dist.is_initialized():
            dist.barrier()
        self.offsets = np.load(offsets_path, mmap_mode="r")
        self.indices = np.load(indices_path, mmap_mode="r")

    def __len__(self) -> int:
        return int(self.offsets[-1])

    def _resolve(self, idx: int) -> Tuple[MemmapDataset, int]:
        p = int(self.indices[idx])
        x = int(np.searchsorted(self.offsets, p, side="right"))
        return self.memmap_datasets[x], (p if x == 0 else p - int(self.offsets[x - 1]))

    def __getitem__(self, idx: int):
        ds, i = self._resolve(idx)
        return ds[i]

    def get_chunk(self, idx: int, seq_offset: int, seq_length: int):
        ds, i = self._resolve(idx)
        return ds.get_chunk(i, seq_offset, seq_length)


class SyntheticDataset:
    """Uniform token ids in ``[0, vocab)``; sequence ``idx`` is a pure function of ``(seed, idx)``."""

    def __init__(self, vocab_size: int, sequence_length: int, seed: int = 0, length: int = 1 << 40):
        self.vocab_size, self.sequence_length, self.seed, self.length = vocab_size, sequence_length, seed, length

    def __len__(self) -> int:
        return self.length

    def _sequence(self, idx: int) -> np.ndarray:
        rng = np.random.default_rng([self.seed, int(idx)])
        return rng.integers(0, self.vocab_size, self.sequence_length + 1, dtype=np.int64)

    def __getitem__(self, idx: int):
        return self.get_chunk(idx, 0, self.sequence_length)

    def get_chunk(self, idx: int, seq_offset: int, seq_length: int):
        seq = self._sequence(idx)
        w = seq[seq_offset:seq_offset + seq_length + 1]
        return torch.from_numpy(w[:-1].copy()), torch.from_numpy(w[1:].copy())
