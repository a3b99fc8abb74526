"""Hash helpers (reference: src/util/hash.zig:7-76): SHA-256 of buffers and files with hex
and verify, a 64-bit xxHash, a 64-bit mix of two hashes, and a string hash."""
from __future__ import annotations

import hashlib

_M64 = (1 << 64) - 1
_P1, _P2, _P3, _P4, _P5 = (11400714785074694791, 14029467366897019727, 1609587929392839161,
                          9650029242287828579, 2870177450012600261)


def sha256(data: bytes) -> bytes:
    return hashlib.sha256(data).digest()


def sha256_file(path, chunk: int = 1 << 20) -> bytes:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.digest()


def to_hex(digest: bytes) -> str:
    return digest.hex()


def verify(data: bytes, expected: bytes) -> bool:
    return sha256(data) == expected


def _rotl(x, r):
    return ((x << r) | (x >> (64 - r))) & _M64


def _round(acc, inp):
    return (_rotl((acc + inp * _P2) & _M64, 31) * _P1) & _M64


def _merge(acc, val):
    return ((acc ^ _round(0, val)) * _P1 + _P4) & _M64


def xxhash64(data: bytes, seed: int = 0) -> int:
    n, i = len(data), 0
    if n >= 32:
        v = [(seed + _P1 + _P2) & _M64, (seed + _P2) & _M64, seed & _M64, (seed - _P1) & _M64]
        while i + 32 <= n:
            for j in range(4):
                v[j] = _round(v[j], int.from_bytes(data[i + 8 * j:i + 8 * j + 8], "little"))
            i += 32
        h = (_rotl(v[0], 1) + _rotl(v[1], 7) + _rotl(v[2], 12) + _rotl(v[3], 18)) & _M64
        for j in range(4):
            h = _merge(h, v[j])
    else:
        h = (seed + _P5) & _M64
    h = (h + n) & _M64
    while i + 8 <= n:
        h ^= _round(0, int.from_bytes(data[i:i + 8], "little"))
        h = (_rotl(h, 27) * _P1 + _P4) & _M64
        i += 8
    if i + 4 <= n:
        h ^= (int.from_bytes(data[i:i + 4], "little") * _P1) & _M64
        h = (_rotl(h, 23) * _P2 + _P3) & _M64
        i += 4
    while i < n:
        h ^= (data[i] * _P5) & _M64
        h = (_rotl(h, 11) * _P1) & _M64
        i += 1
    h ^= h >> 33
    h = (h * _P2) & _M64
    h ^= h >> 29
    h = (h * _P3) & _M64
    h ^= h >> 32
    return h


def combine_hash(a: int, b: int) -> int:
    """hash.zig:65-67 style mix: a ^ (b + golden + (a << 6) + (a >> 2))."""
    return (a ^ ((b + 0x9E3779B97F4A7C15 + ((a << 6) & _M64) + (a >> 2)) & _M64)) & _M64


def hash_string(s: str) -> int:
    return xxhash64(s.encode())
