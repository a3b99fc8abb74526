"""ZeRO stages on the segment ownership layout of ``optim.flat.FlatParams``.

``runtime.zero_stage`` (src/util/config.zig:491,511; the shard arithmetic it stands for is
``ZeroConfig`` / ``ownsParameter`` in src/tensor/sharding.zig:289-355, which nothing in the
reference consults) selects how much of a data-parallel replica's state is partitioned:

* stage 1: optimizer state.  Gradients are reduce-scattered, the owned shard is updated and
  the parameters are all-gathered by ONE kernel after the backward pass
  (``FusedComm.zero_step``).
* stage 2: gradients too.  The reduce-scatter runs bucket by bucket (one transformer block per
  bucket) on a side stream while the backward pass of the last micro-batch is still going
  (``BucketReducer``), so after the backward pass only the norm exchange, the update and the
  parameter all-gather remain.
* stage 3: parameters too (FSDP).  The update leaves the block matrices as row shards; the
  all-gather of ``w_qkv`` (+ ``w_o``) and ``w_up`` (+ ``w_down``) happens inside the first
  GEMM that consumes them after the step (``WeightGather``: every CTA of the GEMM kernel first
  pulls its few 32 KB chunks of the peers' row shards over NVLink, then multiplies, local rows
  first; the gather runs at link rate and is over while the local tiles are being computed).
  The gathered copy is kept for the remaining micro-batches and the backward pass of the step.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import _lib


class BucketReducer:
    """Launches the per-bucket gradient reduce-scatter from tensor hooks on the inputs of the
    transformer blocks during the backward pass of a step's last micro-batch."""

    def __init__(self, comm, flat, block_prefixes, ctas: int = 24):
        self.comm, self.flat, self.ctas = comm, flat, ctas
        self.stream = torch.cuda.Stream()
        nr = len(flat.ranges)
        covered = [False] * nr
        self.buckets = []  # per block: (r0, r1)
        for pre in block_prefixes:
            idx = [i for i, r in enumerate(flat.ranges)
                   if r.names and all(n.startswith(pre) for n in r.names)]
            if not idx:
                self.buckets.append(None)
                continue
            r0, r1 = min(idx), max(idx) + 1
            if idx != list(range(r0, r1)):
                raise ValueError(f"the ranges of {pre} are not contiguous")
            for i in idx:
                covered[i] = True
            self.buckets.append((r0, r1))
        # whatever no block bucket covers (embeddings, LM head, the run of vectors) is reduced
        # after the backward pass, in maximal contiguous runs
        self.rest = []
        i = 0
        while i < nr:
            if covered[i]:
                i += 1
                continue
            j = i
            while j < nr and not covered[j]:
                j += 1
            self.rest.append((i, j))
            i = j
        self.armed = False

    def block_hook(self, block_index: int, grad):
        """Tensor hook on the input of block ``block_index``: every gradient of that block's
        parameters has been launched on the current stream."""
        if self.armed and self.buckets[block_index] is not None:
            self._launch(*self.buckets[block_index])
        return grad

    def _launch(self, r0, r1):
        ev = torch.cuda.Event()
        ev.record()
        self.stream.wait_event(ev)
        self.comm.bucket_reduce(self.flat, r0, r1, self.stream, self.ctas)

    def finish(self):
        """After the backward pass: reduce what the block buckets left, then make the current
        stream wait for all reductions."""
        for r0, r1 in self.rest:
            self._launch(r0, r1)
        torch.cuda.current_stream().wait_stream(self.stream)
        self.armed = False


class WeightGather:
    """The deferred all-gather of one row-sharded weight matrix (and, in the same launch, of a
    second tensor that a later GEMM of the block needs), fused into the GEMM that first
    consumes the weight after an optimizer step."""

    def __init__(self, comm, flat, name: str, extra_name: str | None = None, copy_ctas: int = -1):
        self.comm, self.flat = comm, flat
        seg = flat.segment(name)
        self.N, self.K = seg.shape
        world = comm.world
        rows = self.N // world
        if self.N % world or (rows * self.K * 2) % 16:
            raise ValueError(f"{name}: {self.N} rows do not split over {world} ranks")
        self.blk_rows = math.gcd(rows, 64)
        self.table = flat.params_symm.table(seg.offset * 2)
        self.flags = torch.zeros(self.N // self.blk_rows, dtype=torch.int32, device=flat.device)
        self.calls = 0
        self.pending = False
        self.copy_ctas = copy_ctas
        self.extra_table, self.extra_bytes = None, 0
        if extra_name is not None:
            seg2 = flat.segment(extra_name)
            if seg2.numel % world or (seg2.numel * 2 // world) % 16:
                raise ValueError(f"{extra_name} does not split over {world} ranks")
            self.extra_table = flat.params_symm.table(seg2.offset * 2)
            self.extra_bytes = seg2.numel * 2 // world
        self.segments = [name] + ([extra_name] if extra_name else [])

    def gemm(self, x2: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``x2 @ W^T (+ residual)`` with W's row shards pulled from the peers inside the
        kernel; afterwards the local copy of W (and of the extra tensor) is complete."""
        M, K = x2.shape
        assert K == self.K and x2.dtype == torch.bfloat16 and x2.stride(1) == 1
        out = torch.empty(M, self.N, dtype=torch.bfloat16, device=x2.device)
        self.calls += 1
        dev = x2.device
        _lib.check(_lib.lib().ceo_ag_gemm_bf16(
            self.table, 2, x2.data_ptr(), out.data_ptr(), M, self.N, K, x2.stride(0),
            out.stride(0), 0, 0, 0, 1.0, _lib.ptr(residual),
            residual.stride(0) if residual is not None else 0, self.flags.data_ptr(), self.calls,
            self.comm.rank, self.comm.world, self.copy_ctas, self.blk_rows, self.extra_table,
            self.extra_bytes, _lib.status_word(dev).data_ptr(), _lib.stream()),
            "ceo_ag_gemm_bf16")
        self.pending = False
        return out

    def materialize(self):
        """The same gather without a GEMM (library all-gather, in place): for checkpoints and
        evaluation between steps."""
        if not self.pending:
            return
        f, w, r = self.flat, self.comm.world, self.comm.rank
        for name in self.segments:
            seg = f.segment(name)
            full = f.params[seg.offset:seg.offset + seg.numel]
            n = seg.numel // w
            dist.all_gather_into_tensor(full, full[r * n:(r + 1) * n], group=self.comm.group)
        self.pending = False


def attach_weight_gathers(model, comm, flat) -> list:
    """Stage 3: marks the four matrices of every block as shards-at-rest (the optimizer keeps
    their updated values local) and attaches the fused gathers to ``w_qkv`` and ``w_up``."""
    gathers = []
    for i, blk in enumerate(model.blocks):
        pre = f"blocks.{i}."
        pairs = [(blk.efla.w_qkv, pre + "efla.w_qkv", pre + "efla.w_o"),
                 (blk.mlp.w_up, pre + "mlp.w_up", pre + "mlp.w_down")]
        for param, name, extra in pairs:
            try:
                ri, rx = flat.range_of(name), flat.range_of(extra)
            except KeyError:
                continue
            if len(flat.ranges[ri].names) != 1 or len(flat.ranges[rx].names) != 1:
                continue  # not row-sharded on this world size: stays gathered by the optimizer
            g = WeightGather(comm, flat, name, extra)
            flat.ranges[ri].gather = False
            flat.ranges[rx].gather = False
            param.fsdp_gather = g
            gathers.append(g)
    return gathers
