"""Memory-layout vocabulary (reference: src/tensor/layout.zig:4-158): layout names, padding
rules, tensor-core tile constants and a device memory pool.

The reference's tile constants (128x128x64, "WGMMA 64x64x32") are used by no kernel
(layout.zig:100-113) and its pool's ``allocate`` returns NotImplemented (116-158).  Here the
constants are the ones ``csrc/gemm_tcgen05.cu`` is built with and the pool is a real bump
allocator over one device buffer (used for step-scoped workspaces).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import torch


class Layout(Enum):
    ROW_MAJOR = "row_major"          # (rows, K) with K contiguous: the K-major GEMM operand
    COL_MAJOR = "col_major"          # (K, rows) with rows contiguous: the MN-major operand
    BTHD = "bthd"                    # (batch, time, heads, head_dim): q/k/v/o
    BHTD = "bhtd"
    BHCDD = "bhcdd"                  # (batch, heads, chunks, d, d): per-chunk EFLA states


@dataclass(frozen=True)
class TensorCoreTiles:
    """Tile shape of the tcgen05 GEMM: one CTA computes 128x256 with K blocks of 64; one
    tcgen05.mma instruction is 128x256x16 for bf16."""
    M: int = 128
    N: int = 256
    K: int = 64
    MMA_K: int = 16
    STAGES: int = 4
    TMEM_COLUMNS: int = 512
    SWIZZLE_BYTES: int = 128


@dataclass(frozen=True)
class PaddingStrategy:
    multiple: int = 8  # elements; 16 bytes of bf16, the TMA row-stride granule

    def pad(self, n: int) -> int:
        return pad_dimension(n, self.multiple)


def pad_dimension(n: int, multiple: int) -> int:
    if multiple <= 0:
        raise ValueError("multiple must be positive")
    return (n + multiple - 1) // multiple * multiple


def optimal_leading_dimension(cols: int, elem_bytes: int = 2) -> int:
    """Smallest leading dimension >= cols whose row stride is a multiple of 16 bytes (a TMA
    requirement) and not a multiple of 512 bytes... unless cols already is (padding a dense
    power-of-two matrix would cost more bandwidth than the bank conflicts it avoids)."""
    return pad_dimension(cols, max(1, 16 // elem_bytes))


class MemoryPool:
    """Bump allocator over one device buffer; ``reset`` frees everything at once."""

    def __init__(self, nbytes: int, device="cuda", alignment: int = 256):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.alignment = alignment
        self.offset = 0
        self.peak = 0

    def allocate(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        start = (self.offset + self.alignment - 1) // self.alignment * self.alignment
        if start + nb > self.buf.numel():
            raise MemoryError(f"pool exhausted: need {nb} bytes at {start} of {self.buf.numel()}")
        self.offset = start + nb
        self.peak = max(self.peak, self.offset)
        return self.buf[start:start + nb].view(dtype).view(*shape)

    def reset(self):
        self.offset = 0

    def used(self) -> int:
        return self.offset
