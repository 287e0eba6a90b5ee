"""Synthetic token source: uniform-random ids over the vocabulary, generated on the host into
pinned memory so a training step pays a real host->device copy, with a per-rank seed."""
from __future__ import annotations

from typing import Iterator, Optional

import torch


class SyntheticTokens:
    def __init__(self, vocab: int, batch: int, seq_len: int, seed: int = 0, rank: int = 0,
                 pin: bool = True, pool: int = 8, exclude: Optional[int] = None) -> None:
        g = torch.Generator().manual_seed(int(seed) + 1000003 * int(rank))
        self.batches = []
        for _ in range(max(1, pool)):
            t = torch.randint(0, vocab, (batch, seq_len + 1), generator=g, dtype=torch.long)
            if exclude is not None:
                t = torch.where(t.eq(int(exclude)), (t + 1) % vocab, t)
            if pin and torch.cuda.is_available():
                t = t.pin_memory()
            self.batches.append(t)
        self._i = 0

    def next(self) -> torch.Tensor:
        t = self.batches[self._i % len(self.batches)]
        self._i += 1
        return t

    def __iter__(self) -> Iterator[torch.Tensor]:
        while True:
            yield self.next()
