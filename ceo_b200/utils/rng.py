"""Deterministic random number generators (reference: src/util/rng.zig:4-166).

``DeterministicRng``: PCG-XSH-RR 64/32 with ``float`` in [0,1), Box-Muller ``float_norm``,
``int_range``, Fisher-Yates ``shuffle`` and ``fork`` (rng.zig:4-84).  ``DistributedRng``:
four independent streams per rank (data, dropout, init, general) seeded by seed XOR
rank * golden ratio (rng.zig:87-134).  ``PhiloxRng``: a counter-based Philox-4x32-10
generator whose output depends only on (seed, counter), so any rank or thread can draw the
same number without shared state (the reference's is a simplified stand-in: rng.zig:137-166).
"""
from __future__ import annotations

import math

_M64 = (1 << 64) - 1
_M32 = (1 << 32) - 1
_PCG_MULT = 6364136223846793005
_GOLDEN = 0x9E3779B97F4A7C15


class DeterministicRng:
    def __init__(self, seed: int, stream: int = 0):
        self.inc = ((stream << 1) | 1) & _M64
        self.state = 0
        self.next_u32()
        self.state = (self.state + (seed & _M64)) & _M64
        self.next_u32()
        self._spare = None

    def next_u32(self) -> int:
        old = self.state
        self.state = (old * _PCG_MULT + self.inc) & _M64
        xorshifted = (((old >> 18) ^ old) >> 27) & _M32
        rot = old >> 59
        return ((xorshifted >> rot) | (xorshifted << ((-rot) & 31))) & _M32

    def next_u64(self) -> int:
        return (self.next_u32() << 32) | self.next_u32()

    def float(self) -> float:
        return self.next_u32() / 4294967296.0

    def float_norm(self) -> float:
        if self._spare is not None:
            s, self._spare = self._spare, None
            return s
        u1 = max(self.float(), 1e-12)
        u2 = self.float()
        r = math.sqrt(-2.0 * math.log(u1))
        self._spare = r * math.sin(2 * math.pi * u2)
        return r * math.cos(2 * math.pi * u2)

    def int_range(self, lo: int, hi: int) -> int:
        """Uniform integer in [lo, hi) without modulo bias."""
        span = hi - lo
        if span <= 0:
            raise ValueError("empty range")
        limit = (1 << 32) - ((1 << 32) % span)
        while True:
            x = self.next_u32()
            if x < limit:
                return lo + x % span

    def shuffle(self, items: list) -> None:
        for i in range(len(items) - 1, 0, -1):
            j = self.int_range(0, i + 1)
            items[i], items[j] = items[j], items[i]

    def fork(self) -> "DeterministicRng":
        return DeterministicRng(self.next_u64(), self.next_u64() >> 1)

    def state_bytes(self) -> bytes:
        return self.state.to_bytes(8, "little") + self.inc.to_bytes(8, "little")

    @classmethod
    def from_state_bytes(cls, b: bytes) -> "DeterministicRng":
        r = cls.__new__(cls)
        r.state = int.from_bytes(b[:8], "little")
        r.inc = int.from_bytes(b[8:16], "little")
        r._spare = None
        return r


class DistributedRng:
    STREAMS = ("data", "dropout", "init", "general")

    def __init__(self, seed: int, rank: int):
        base = (seed ^ ((rank * _GOLDEN) & _M64)) & _M64
        self.rank = rank
        self.streams = {n: DeterministicRng(base, stream=i + 1 + 4 * rank)
                        for i, n in enumerate(self.STREAMS)}

    def __getitem__(self, name: str) -> DeterministicRng:
        return self.streams[name]

    def state_bytes(self) -> bytes:
        return b"".join(self.streams[n].state_bytes() for n in self.STREAMS)

    def load_state_bytes(self, b: bytes) -> None:
        for i, n in enumerate(self.STREAMS):
            self.streams[n] = DeterministicRng.from_state_bytes(b[16 * i:16 * i + 16])


class PhiloxRng:
    _M0, _M1 = 0xD2511F53, 0xCD9E8D57
    _W0, _W1 = 0x9E3779B9, 0xBB67AE85

    def __init__(self, seed: int):
        self.key = (seed & _M32, (seed >> 32) & _M32)

    def block(self, counter: int) -> tuple:
        """Four 32-bit outputs for a 128-bit counter."""
        c = [(counter >> (32 * i)) & _M32 for i in range(4)]
        k0, k1 = self.key
        for _ in range(10):
            p0 = self._M0 * c[0]
            p1 = self._M1 * c[2]
            c = [((p1 >> 32) ^ c[1] ^ k0) & _M32, p1 & _M32,
                 ((p0 >> 32) ^ c[3] ^ k1) & _M32, p0 & _M32]
            k0 = (k0 + self._W0) & _M32
            k1 = (k1 + self._W1) & _M32
        return tuple(c)

    def uniform(self, counter: int) -> float:
        return self.block(counter)[0] / 4294967296.0
