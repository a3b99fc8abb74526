"""Seeded synthetic token streams: i.i.d. uniform or Zipf(s) over the vocabulary.

Used by the benchmark configurations (random-init weights, no dataset on disk) and by
``data.synthetic`` in the YAML schema.  The Zipf sampler draws ranks by inverting the
cumulative distribution p(r) ~ r^-s over a fixed vocabulary, so it is exact for any s > 0.
"""
from __future__ import annotations

import numpy as np
import torch


class SyntheticTokens:
    def __init__(self, vocab_size: int, kind: str = "zipf", s: float = 1.1, seed: int = 0,
                 rank: int = 0):
        if kind not in ("uniform", "zipf"):
            raise ValueError(f"synthetic kind must be uniform or zipf, got {kind!r}")
        self.vocab, self.kind = vocab_size, kind
        self.rng = np.random.default_rng([seed, rank])
        if kind == "zipf":
            w = np.arange(1, vocab_size + 1, dtype=np.float64) ** (-s)
            self.cdf = np.cumsum(w / w.sum())

    def sample(self, n: int) -> np.ndarray:
        if self.kind == "uniform":
            return self.rng.integers(0, self.vocab, size=n, dtype=np.int64)
        u = self.rng.random(n)
        return np.minimum(np.searchsorted(self.cdf, u), self.vocab - 1).astype(np.int64)

    def batch(self, batch: int, seq_len: int, pin: bool = False):
        """(tokens, targets), each (batch, seq_len) int64: targets are the next tokens."""
        x = torch.from_numpy(self.sample(batch * (seq_len + 1)).reshape(batch, seq_len + 1))
        tok, tgt = x[:, :-1].contiguous(), x[:, 1:].contiguous()
        if pin and torch.cuda.is_available():
            tok, tgt = tok.pin_memory(), tgt.pin_memory()
        return tok, tgt
