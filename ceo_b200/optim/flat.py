"""Flat parameter storage for sharded mixed-precision training.

All bf16 parameters of a model become views into ONE contiguous bf16 buffer, with a
matching fp32 gradient buffer (each parameter gets ``.main_grad``, the view the GEMM
epilogues accumulate into) and, for the slice a rank owns, fp32 master weights and
optimizer moments.  With ``world > 1`` the buffer is padded so it splits evenly and rank
r owns ``[r*shard, (r+1)*shard)``: gradients are reduce-scattered onto the owner, the
owner updates its slice and the bf16 slices are all-gathered - ZeRO / FSDP sharding of
gradients and optimizer state (the reference only describes this: ``ZeroConfig`` and
``ownsParameter`` in src/tensor/sharding.zig:289-355).

Parameters that are not bf16 (the scalar ``beta_param``) stay outside the flat buffer in a
small fp32 side group that every rank updates identically after an all-reduce.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

ALIGN = 256  # elements; keeps every rank's slice 512-byte aligned


@dataclass
class Segment:
    name: str
    offset: int
    numel: int
    shape: tuple
    decay: bool


class FlatParams:
    def __init__(self, model: torch.nn.Module, world: int = 1, rank: int = 0,
                 grad_dtype: torch.dtype = torch.float32, alloc=None):
        """``alloc(numel, dtype) -> (tensor, handle)`` places the parameter and gradient
        buffers in peer-mapped memory (``FusedComm.alloc``); default: ordinary tensors."""
        self.world, self.rank = world, rank
        named = [(n, p) for n, p in model.named_parameters()]
        flat_named = [(n, p) for n, p in named if p.dtype in (torch.bfloat16, torch.float32)
                      and p.dim() >= 1 and p.numel() > 1]
        self.side = [(n, p) for n, p in named if not any(p is q for _, q in flat_named)]
        if not flat_named:
            raise ValueError("model has no parameters")
        dev = flat_named[0][1].device
        self.device = dev
        self.param_dtype = flat_named[0][1].dtype
        # matrices first, vectors last: the decayed part is one contiguous range
        order = sorted(range(len(flat_named)), key=lambda i: (flat_named[i][1].dim() < 2, i))
        self.segments: list[Segment] = []
        off = 0
        for i in order:
            n, p = flat_named[i]
            self.segments.append(Segment(n, off, p.numel(), tuple(p.shape), p.dim() >= 2))
            off += (p.numel() + 7) // 8 * 8
        self.decay_end = max((s.offset + (s.numel + 7) // 8 * 8 for s in self.segments if s.decay),
                             default=0)
        # the decay boundary must not split a rank's slice unevenly for the kernels' sake:
        # kernels take (offset, length) ranges, so any boundary works.
        unit = ALIGN * world
        self.total = (off + unit - 1) // unit * unit
        self.shard = self.total // world
        self.params_symm = self.grads_symm = None
        if alloc is not None:
            self.params, self.params_symm = alloc(self.total, self.param_dtype)
            self.grads, self.grads_symm = alloc(self.total, grad_dtype)
        else:
            self.params = torch.zeros(self.total, dtype=self.param_dtype, device=dev)
            self.grads = torch.zeros(self.total, dtype=grad_dtype, device=dev)
        self._by_name = {}
        for seg, i in zip(self.segments, order):
            n, p = flat_named[i]
            view = self.params[seg.offset:seg.offset + seg.numel].view(seg.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grads[seg.offset:seg.offset + seg.numel].view(seg.shape)
            p.grad_touched = False
            self._by_name[n] = p
        lo = rank * self.shard
        self.lo, self.hi = lo, lo + self.shard
        self.master = self.params[lo:self.hi].float()
        self.state: dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ helpers
    def owned(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.lo:self.hi]

    def owned_ranges(self):
        """[(start, stop, decay)] in local (shard-relative) coordinates."""
        out = []
        d0, d1 = max(self.lo, 0), min(self.hi, self.decay_end)
        if d1 > d0:
            out.append((d0 - self.lo, d1 - self.lo, True))
        n0, n1 = max(self.lo, self.decay_end), self.hi
        if n1 > n0:
            out.append((n0 - self.lo, n1 - self.lo, False))
        return out

    def buffer(self, key: str) -> torch.Tensor:
        if key not in self.state:
            self.state[key] = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
        return self.state[key]

    def param(self, name: str):
        return self._by_name[name]

    def zero_grads(self):
        self.grads.zero_()
        for _, p in self.side:
            p.grad = None

    def numel(self) -> int:
        return sum(s.numel for s in self.segments)

    # ------------------------------------------------------ checkpoint (de)serialisation
    def optimizer_state(self) -> dict:
        return {"master": self.master, **self.state}

    def load_optimizer_state(self, st: dict):
        self.master.copy_(st["master"])
        for k, v in st.items():
            if k != "master":
                self.buffer(k).copy_(v)

    def refresh_master(self):
        """Re-derive the fp32 master slice from the (just loaded) bf16 parameters."""
        self.master.copy_(self.params[self.lo:self.hi].float())
