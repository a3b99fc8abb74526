"""Flat parameter storage for sharded mixed-precision training.

All bf16 parameters of a model become views into ONE contiguous bf16 buffer, with a
matching fp32 gradient buffer (each parameter gets ``.main_grad``, the view the GEMM
epilogues accumulate into) and, for the part a rank owns, fp32 master weights and
optimizer moments - ZeRO / FSDP sharding of gradients and optimizer state (the reference
only describes this: ``ZeroConfig`` and ``ownsParameter`` in src/tensor/sharding.zig:289-355).

Two ownership layouts:

* ``contiguous``: the buffer is padded so it splits evenly and rank r owns
  ``[r*shard, (r+1)*shard)``.  This is what the library collectives (reduce-scatter /
  all-gather of equal contiguous chunks) need.
* ``segment``: every matrix whose rows divide evenly is split by rows, rank r owning rows
  ``[r*rows/world, (r+1)*rows/world)`` of EACH matrix; whatever is left (vectors, odd
  matrices) forms contiguous runs that are split evenly.  A bucket of a few matrices (one
  transformer block) is then reduced by all ranks at once, and a weight's row shards are what
  the all-gather fused into its consuming GEMM pulls.  The rank's master weights and moments
  live in shard-local buffers, range after range (``ranges``).

Parameters that are not bf16 (the scalar ``beta_param``) stay outside the flat buffer in a
small fp32 side group that every rank updates identically after an all-reduce.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

ALIGN = 256  # elements; keeps every rank's slice 512-byte aligned
SEG_PAD = 64  # every segment starts on a multiple of this many elements (any world <= 8)


@dataclass
class Segment:
    name: str
    offset: int
    numel: int
    shape: tuple
    decay: bool


@dataclass
class OwnedRange:
    """Rank r owns flat elements [goff + r*len, goff + (r+1)*len); they sit at
    [loff, loff+len) of the shard-local buffers."""
    goff: int
    len: int
    loff: int
    gather: bool = True
    names: tuple = ()


def _padded(n: int) -> int:
    return (n + SEG_PAD - 1) // SEG_PAD * SEG_PAD


def build_ranges(segments, total: int, world: int, layout: str) -> list[OwnedRange]:
    """The ownership map of a flat buffer (the same for every rank)."""
    if layout == "contiguous":
        return [OwnedRange(0, total // world, 0, True, tuple(s.name for s in segments))]
    if world not in (1, 2, 4, 8):
        raise ValueError("the segment layout needs a power-of-two world size of at most 8")
    out: list[OwnedRange] = []
    loff = 0
    run_start, run_names = None, []

    def flush(end):
        nonlocal run_start, run_names, loff
        if run_start is not None and end > run_start:
            ln = (end - run_start) // world
            out.append(OwnedRange(run_start, ln, loff, True, tuple(run_names)))
            loff += ln
        run_start, run_names = None, []

    for s in segments:
        rows = s.shape[0] if len(s.shape) == 2 else 0
        if rows and rows % world == 0 and s.numel % (8 * world) == 0:
            flush(s.offset)
            ln = s.numel // world
            out.append(OwnedRange(s.offset, ln, loff, True, (s.name,)))
            loff += ln
            # (padding behind the matrix, if any, belongs to nobody: it is never read)
        else:
            if run_start is None:
                run_start = s.offset
            run_names.append(s.name)
    flush(total)
    return out


class FlatParams:
    def __init__(self, model: torch.nn.Module, world: int = 1, rank: int = 0,
                 grad_dtype: torch.dtype = torch.float32, alloc=None,
                 layout: str = "contiguous"):
        """``alloc(numel, dtype) -> (tensor, handle)`` places the parameter and gradient
        buffers in peer-mapped memory (``FusedComm.alloc``); default: ordinary tensors."""
        if layout not in ("contiguous", "segment"):
            raise ValueError(layout)
        self.world, self.rank, self.layout = world, rank, layout
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
            off += _padded(p.numel())
        self.decay_end = max((s.offset + _padded(s.numel) for s in self.segments if s.decay),
                             default=0)
        unit = ALIGN * world
        self.total = (off + unit - 1) // unit * unit
        self.ranges = build_ranges(self.segments, self.total, world, layout)
        self.shard = sum(r.len for r in self.ranges)
        self.params_symm = self.grads_symm = None
        if alloc is not None:
            self.params, self.params_symm = alloc(self.total, self.param_dtype)
            self.grads, self.grads_symm = alloc(self.total, grad_dtype)
        else:
            self.params = torch.zeros(self.total, dtype=self.param_dtype, device=dev)
            self.grads = torch.zeros(self.total, dtype=grad_dtype, device=dev)
        self._by_name = {}
        self._seg_by_name = {}
        for seg, i in zip(self.segments, order):
            n, p = flat_named[i]
            view = self.params[seg.offset:seg.offset + seg.numel].view(seg.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grads[seg.offset:seg.offset + seg.numel].view(seg.shape)
            p.grad_touched = False
            self._by_name[n] = p
            self._seg_by_name[n] = seg
        # contiguous layout: [lo, hi) is the owned slice
        self.lo = rank * self.shard if layout == "contiguous" else 0
        self.hi = self.lo + self.shard if layout == "contiguous" else 0
        self.master = torch.empty(self.shard, dtype=torch.float32, device=dev)
        self.refresh_master()
        self.state: dict[str, torch.Tensor] = {}
        self._ranges_dev = None

    # ------------------------------------------------------------------ helpers
    def owned_views(self, t: torch.Tensor):
        """The slices of a full flat tensor this rank owns, in shard-local order."""
        return [t[r.goff + self.rank * r.len:r.goff + (self.rank + 1) * r.len] for r in self.ranges]

    def owned(self, t: torch.Tensor) -> torch.Tensor:
        v = self.owned_views(t)
        return v[0] if len(v) == 1 else torch.cat(v)

    def owned_ranges(self):
        """[(start, stop, decay)] in local (shard-relative) coordinates (contiguous layout)."""
        assert self.layout == "contiguous"
        out = []
        d0, d1 = max(self.lo, 0), min(self.hi, self.decay_end)
        if d1 > d0:
            out.append((d0 - self.lo, d1 - self.lo, True))
        n0, n1 = max(self.lo, self.decay_end), self.hi
        if n1 > n0:
            out.append((n0 - self.lo, n1 - self.lo, False))
        return out

    def ranges_device(self) -> torch.Tensor:
        """The ownership map as the device record array ``ceo_zero_step`` reads
        ({int64 goff, len, loff; int32 gather, pad} per range)."""
        if self._ranges_dev is None or self._ranges_dev[1] != [r.gather for r in self.ranges]:
            rows = []
            for r in self.ranges:
                rows.append([r.goff, r.len, r.loff, int(r.gather)])  # low int32 = gather, high = 0
            t = torch.tensor(rows, dtype=torch.int64)
            self._ranges_dev = (t.to(self.device), [r.gather for r in self.ranges])
        return self._ranges_dev[0]

    def range_of(self, name: str) -> int:
        for i, r in enumerate(self.ranges):
            if name in r.names:
                return i
        raise KeyError(name)

    def buffer(self, key: str) -> torch.Tensor:
        if key not in self.state:
            self.state[key] = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
        return self.state[key]

    def param(self, name: str):
        return self._by_name[name]

    def segment(self, name: str) -> Segment:
        return self._seg_by_name[name]

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
        """Re-derive the fp32 master shard from the (just loaded) bf16 parameters."""
        off = 0
        for v in self.owned_views(self.params):
            self.master[off:off + v.numel()].copy_(v.float())
            off += v.numel()

    def layout_info(self) -> dict:
        return {"layout": self.layout, "world": self.world, "total": self.total}

    def reshard(self, parts: list, saved: dict) -> torch.Tensor:
        """Rebuilds this rank's shard of a flat-shard tensor (master weights or a moment) from
        the shards ``parts[r]`` every rank of another run saved with the ownership map
        ``saved`` = its ``layout_info()``."""
        sw, slay = int(saved["world"]), saved["layout"]
        stotal = int(saved.get("total", self.total))
        if slay == "contiguous":
            # the saved buffer may have been padded for another world size
            shard = parts[0].numel()
            stotal = shard * sw
        full = torch.zeros(max(stotal, self.total), dtype=parts[0].dtype)
        old = build_ranges(self.segments, stotal, sw, slay)
        for r in range(sw):
            src = parts[r].reshape(-1).cpu()
            for rg in old:
                full[rg.goff + r * rg.len:rg.goff + (r + 1) * rg.len] = src[rg.loff:rg.loff + rg.len]
        mine = [full[rg.goff + self.rank * rg.len:rg.goff + (self.rank + 1) * rg.len]
                for rg in self.ranges]
        return torch.cat(mine) if len(mine) > 1 else mine[0].clone()
