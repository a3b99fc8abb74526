"""Process-group plumbing and the library-collective (NCCL / gloo) baseline.

One process per GPU, ``torch.distributed`` for rendezvous; ``Comm`` exposes the
collectives the sharded optimizer and the parallel layers need.  The same interface is
implemented by ``FusedComm`` (``fused.py``) with in-kernel peer access over NVLink; this
class is the NCCL baseline those kernels are measured against and the CPU (gloo) path of
the multi-process tests.

Counterpart of the reference's ProcessGroup / NcclCollectives wrappers
(src/runtime/main.zig:10-138, src/runtime/nccl.zig:214-345): all-reduce, reduce,
broadcast, reduce-scatter, all-gather, send/recv, all-to-all, barrier, with the same
world_size == 1 short-circuits (main.zig:66-79, 92-94).
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def init_distributed(backend: str | None = None, timeout_s: float = 600.0):
    """Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* from the environment (torchrun).
    Returns (rank, world, local_rank).  A single process needs no rendezvous."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1:
        return 0, 1, 0
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


class Comm:
    """Collectives over one process group (library implementation)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._rs_out = None

    # ---- reductions -----------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM):
        if self.world > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    def reduce(self, t, dst: int, op=dist.ReduceOp.SUM):
        if self.world > 1:
            dist.reduce(t, dst=self._global(dst), op=op, group=self.group)
        return t

    def reduce_scatter(self, buf: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
        """Sum ``buf`` (same length on every rank) across ranks; returns this rank's slice
        [lo, hi) of the sum."""
        if self.world == 1:
            return buf[lo:hi]
        if buf.device.type == "cpu":  # gloo has no reduce_scatter_tensor
            dist.all_reduce(buf, group=self.group)
            return buf[lo:hi]
        out = buf[lo:hi]
        dist.reduce_scatter_tensor(out, buf, group=self.group)
        return out

    # ---- gathers / broadcasts -----------------------------------------------------------
    def all_gather(self, buf: torch.Tensor, lo: int, hi: int):
        """Every rank contributes buf[lo:hi]; afterwards ``buf`` is complete everywhere."""
        if self.world == 1:
            return buf
        if buf.device.type == "cpu":
            parts = [torch.empty(hi - lo, dtype=buf.dtype) for _ in range(self.world)]
            dist.all_gather(parts, buf[lo:hi].clone(), group=self.group)
            buf.copy_(torch.cat(parts))
            return buf
        dist.all_gather_into_tensor(buf, buf[lo:hi], group=self.group)
        return buf

    def all_gather_cat(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=dim)

    def broadcast(self, t, src: int = 0):
        if self.world > 1:
            dist.broadcast(t, src=self._global(src), group=self.group)
        return t

    def broadcast_segments(self, flat, segs):
        """Segment i of ``segs`` is owned by rank i % world (whole matrices for Muon)."""
        works = []
        for i, s in enumerate(segs):
            view = flat.params[s.offset:s.offset + s.numel]
            works.append(dist.broadcast(view, src=self._global(i % self.world), group=self.group,
                                        async_op=True))
        for w in works:
            w.wait()

    # ---- point to point / all-to-all ---------------------------------------------------
    def send(self, t, dst: int):
        dist.send(t, dst=self._global(dst), group=self.group)

    def recv(self, t, src: int):
        dist.recv(t, src=self._global(src), group=self.group)
        return t

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor):
        if self.world == 1:
            out.copy_(inp)
            return out
        if inp.device.type == "cpu":
            ins = list(inp.chunk(self.world))
            outs = [torch.empty_like(c) for c in ins]
            works = []
            for r in range(self.world):
                if r == self.rank:
                    outs[r].copy_(ins[r])
                    continue
                works.append(dist.isend(ins[r].contiguous(), self._global(r), group=self.group))
                works.append(dist.irecv(outs[r], self._global(r), group=self.group))
            for w in works:
                w.wait()
            out.copy_(torch.cat(outs))
            return out
        dist.all_to_all_single(out, inp, group=self.group)
        return out

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)

    def _global(self, group_rank: int) -> int:
        if self.group is None or not dist.is_initialized():
            return group_rank
        return dist.get_global_rank(self.group, group_rank)

    # ---- timing helpers ----------------------------------------------------------------
    def max_over_ranks(self, value: float, device=None) -> float:
        if self.world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64,
                         device=device or ("cuda" if dist.get_backend(self.group) == "nccl"
                                           else "cpu"))
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())
