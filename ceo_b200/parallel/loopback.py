"""Single-GPU stand-ins for the peer tables of the fused collectives.

A kernel that talks to its peers takes a table of ``world`` device pointers.  Here every
entry points into THIS GPU's memory, so one process on one GPU can launch the real kernels
with ``world = 2`` (or more): the "peer" buffers are ordinary local tensors that the caller
fills (a peer's gradients, a peer's weight shard) and the "peer" flag words are local words
that the caller either pre-sets (``signal``) so the kernel's bounded waits are satisfied at
once, or leaves alone so that a wait runs out.  Nothing here waits on another launch: exactly
one kernel runs at a time.

Used for two things that must not involve a second process:
* tests of the time-out path (a flag nobody sets; the kernel must return with a status word
  and leave its state untouched),
* profiler captures of the fused kernels on one GPU (replayed launches need no partner).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib

BIG_EPOCH = 1 << 30  # a flag value every barrier epoch used below compares as "arrived"


def table(tensors) -> ctypes.Array:
    """ctypes array of 8 device pointers (unused entries null) from a list of tensors."""
    ptrs = [t.data_ptr() for t in tensors]
    return (ctypes.c_void_p * 8)(*(ptrs + [None] * (8 - len(ptrs))))


class LoopbackPeers:
    """Flag / slot control blocks for ``world`` pretend ranks, all on the current GPU."""

    def __init__(self, world: int = 2, device=None):
        self.world = world
        self.dev = torch.device(device) if device is not None else \
            torch.device("cuda", torch.cuda.current_device())
        # per pretend rank: 8 flag slots x 8 words, then 8 floats of norm slots, 64 of staging
        self.ctrl = [torch.zeros(1024, dtype=torch.int32, device=self.dev) for _ in range(world)]
        self.epoch = 2

    def flags(self):
        return table(self.ctrl)

    def slots(self):
        return table([c[128:] for c in self.ctrl])  # byte offset 512

    def staging(self):
        return table([c[256:] for c in self.ctrl])  # byte offset 1024

    def signal(self, rank: int = 0):
        """Marks every pretend peer as already arrived at every barrier slot of ``rank``'s
        flag block (for launches that should run through)."""
        self.ctrl[rank][:64] = BIG_EPOCH

    def next_epoch(self) -> int:
        self.epoch += 2
        return self.epoch

    def status(self) -> torch.Tensor:
        return _lib.status_word(self.dev)
