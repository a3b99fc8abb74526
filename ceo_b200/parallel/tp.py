"""Tensor parallelism with sequence-sharded activations: the collectives ride inside the
GEMM kernels (``csrc/gemm_tcgen05.cu``).

* ``ag_gemm``: all-gather of the row-sharded activation fused into the column-parallel GEMM
  (QKV / up projections): copy CTAs pull the peers' shards over NVLink while the remaining
  CTAs multiply, starting with the local rows.
* ``gemm_rs``: row-parallel GEMM (out / down projections) whose epilogue stores each partial
  tile into the owning rank's staging buffer; every rank then reduces its own rows (and adds
  the residual) at the end of the same kernel.
* ``ColumnParallelLinear`` / ``RowParallelLinear``: autograd functions built from the two
  (the backward of one is the other), with NCCL compositions of the same math
  (``impl="nccl"``) as the measured baseline.

The reference only records which dimension of each layer would be split
(src/tensor/sharding.zig:183-222) and has no tensor-parallel execution.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.matmul import gemm
from .symm import SymmetricBuffer


class TPContext:
    """Symmetric workspaces of one tensor-parallel group for activations of up to
    ``max_rows`` (gathered) rows by ``max_cols`` columns."""

    def __init__(self, comm, max_rows: int, max_cols: int, copy_ctas: int = -1):
        self.comm, self.group = comm, comm.group
        self.rank, self.world = comm.rank, comm.world
        self.max_rows, self.max_cols = max_rows, max_cols
        self.copy_ctas = copy_ctas
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        nb = max_rows * max_cols * 2
        # AG destination (rows x K), twice: calls alternate between the halves, so a rank that
        # is already filling in its shard for the next call cannot disturb a peer that is still
        # pulling the previous one (no barrier after the kernel)
        self.gather = SymmetricBuffer(2 * nb, self.group)
        self.gather_half = nb
        # RS staging [world][rows/world][N], twice: successive calls alternate between the two
        # halves (a rank may be one call ahead of a peer that still reduces the previous one)
        self.stage = SymmetricBuffer(2 * nb, self.group)
        self.stage_half = nb
        self.rs_calls = 0
        self.rs_rows = None
        nblk = (max_rows + 127) // 128
        self.counters = SymmetricBuffer(self.world * nblk * 4, self.group)
        self.ag_flags = torch.zeros(nblk, dtype=torch.int32, device=dev)
        self.ag_counter = torch.zeros(1, dtype=torch.int32, device=dev)  # copy-first mode
        self.ag_calls = 0
        self.rs_target = 0
        self.nblk = nblk

    def barrier(self):
        self.comm.device_barrier()

    # ------------------------------------------------------------------ fused ops
    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False,
                out_dtype=torch.bfloat16, keep_gathered: bool = False):
        """``all_gather(x_shard, dim=0) @ w^T``.  x_shard: (M/world, K) bf16; w: (N, K)
        (or (K, N) with ``w_mn``).  Returns C (M, N) [and a copy of the gathered x]."""
        rows, K = x_shard.shape
        M = rows * self.world
        N = w.shape[1] if w_mn else w.shape[0]
        assert M * K * 2 <= self.gather_half and rows % 128 == 0
        self.ag_calls += 1
        half = (self.ag_calls & 1) * self.gather_half
        full = self.gather.view(torch.bfloat16, M * K, half).view(M, K)
        full[self.rank * rows:(self.rank + 1) * rows].copy_(x_shard)
        # every rank's shard is in place - and every rank has finished the call before last,
        # which used this half of the buffer
        self.barrier()
        out = torch.empty(M, N, dtype=out_dtype, device=self.dev)
        remote = (self.world - 1) / self.world * M * K * 2
        if self.copy_ctas < 0 and remote <= 24e6:
            # copy-first: every CTA moves its share of the peers' shards, then computes (local
            # rows first); one counter instead of per-block flags.  Pays while a CTA's share
            # fits its ring of six 32 KB buffers (one NVLink round trip for the whole gather):
            # measured at 2 ranks, 17 MB of weights arrive in 23 us, but 67 MB of activations
            # take 135 us of copy-only time where 8 copy CTAs hide them behind the GEMM
            copy_ctas, flags = -1, self.ag_counter
        else:
            # dedicated copy CTAs, enough of them to keep NVLink busy when the transfer, not
            # the math, is the bound (one copy CTA sustains a few tens of GB/s: six 32 KB bulk
            # copies in flight)
            comm_s = (self.world - 1) / self.world * M * K * 2 / 770e9
            math_s = 2.0 * M * N * K / 1.4e15
            ratio = comm_s / max(math_s, 1e-9)
            base = self.copy_ctas if self.copy_ctas > 0 else 8
            copy_ctas = base if ratio < 0.3 else (16 if ratio < 0.6 else 24)
            flags = self.ag_flags
        L = _lib.lib()
        _lib.check(L.ceo_ag_gemm_bf16(self.gather.table(half), 1, w.data_ptr(), out.data_ptr(), M, N, K,
                                      w.stride(0), out.stride(0), int(w_mn),
                                      int(out_dtype == torch.float32), 0, 1.0, None, 0,
                                      flags.data_ptr(), self.ag_calls, self.rank,
                                      self.world, copy_ctas, 0, None, 0,
                                      _lib.status_word(self.dev).data_ptr(), _lib.stream()),
                   "ceo_ag_gemm_bf16")
        saved = full.clone() if keep_gathered else None
        return (out, saved) if keep_gathered else out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False,
                residual: torch.Tensor | None = None):
        """``reduce_scatter(a @ w^T, dim=0) (+ residual)``.  a: (M, K_local); w: (N, K_local)
        (or (K_local, N) with ``w_mn``); residual / result: (M/world, N) bf16."""
        M, K = a.shape
        N = w.shape[1] if w_mn else w.shape[0]
        rows = M // self.world
        assert M % self.world == 0 and rows % 128 == 0 and M * N * 2 <= self.stage_half
        assert M // 128 <= self.nblk
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=self.dev)
        if self.rs_rows != rows:
            # another row count re-maps the counters: start over behind a barrier (every rank
            # has then consumed what was sent to it)
            self.barrier()
            self.counters.view(torch.int32, self.world * self.nblk).zero_()
            self.barrier()
            self.rs_target, self.rs_rows = 0, rows
        # counters only grow: no reset and no barrier between calls of the same shape
        self.rs_target += 4 * ((N + 255) // 256)
        self.rs_calls += 1
        # more reducer CTAs when the transfer, not the math, bounds the kernel
        comm_s = (self.world - 1) / self.world * M * N * 2 / 770e9
        math_s = 2.0 * M * N * K / 1.4e15
        ratio = comm_s / max(math_s, 1e-9)
        rs_ctas = 24 if ratio < 0.3 else (32 if ratio < 1.0 else 40)
        L = _lib.lib()
        _lib.check(L.ceo_gemm_rs_bf16(a.data_ptr(), w.data_ptr(), M, N, K, a.stride(0),
                                      w.stride(0), 0, int(w_mn), 1.0,
                                      self.stage.table((self.rs_calls & 1) * self.stage_half),
                                      self.counters.table(), self.rs_target, out.data_ptr(),
                                      _lib.ptr(residual),
                                      out.stride(0), self.rank, self.world, rs_ctas,
                                      _lib.status_word(self.dev).data_ptr(), _lib.stream()),
                   "ceo_gemm_rs_bf16")
        return out

    # ------------------------------------------------------- NCCL compositions (baseline)
    def ag_gemm_nccl(self, x_shard, w, *, w_mn=False, out_dtype=torch.bfloat16):
        rows, K = x_shard.shape
        full = torch.empty(rows * self.world, K, dtype=x_shard.dtype, device=self.dev)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        return gemm(full, w, b_mn=w_mn, out_dtype=out_dtype), full

    def gemm_rs_nccl(self, a, w, *, w_mn=False, residual=None):
        part = gemm(a, w, b_mn=w_mn)
        out = torch.empty(part.shape[0] // self.world, part.shape[1], dtype=part.dtype,
                          device=self.dev)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        if residual is not None:
            out = out + residual
        return out

    def close(self):
        for b in (self.gather, self.stage, self.counters):
            b.close()


class _ColumnParallel(torch.autograd.Function):
    """y (M, N_local) = all_gather(x) @ W_local^T; backward: dx = reduce_scatter(dy @ W_local)."""

    @staticmethod
    def forward(ctx, x_shard, weight, tp, impl):
        if impl == "fused":
            y, full = tp.ag_gemm(x_shard, weight, keep_gathered=True)
        else:
            y, full = tp.ag_gemm_nccl(x_shard, weight)
        ctx.save_for_backward(full)
        ctx.wref, ctx.tp, ctx.impl = weight, tp, impl
        return y

    @staticmethod
    def backward(ctx, dy):
        (full,) = ctx.saved_tensors
        w, tp = ctx.wref, ctx.tp
        dy = dy.contiguous()
        # dx_shard = reduce_scatter(dy (M,N_loc) @ W (N_loc,K)):  B operand is W stored (K_c, N_out)
        if ctx.impl == "fused":
            dx = tp.gemm_rs(dy, w, w_mn=True)
        else:
            dx = tp.gemm_rs_nccl(dy, w, w_mn=True)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            gemm(dy, full, a_mn=True, b_mn=True, out=mg, accumulate=True)
            w.grad_touched = True
            return dx, None, None, None
        return dx, gemm(dy, full, a_mn=True, b_mn=True, out_dtype=w.dtype), None, None


class _RowParallel(torch.autograd.Function):
    """y_shard (M/world, N) = reduce_scatter(x (M, K_local) @ W_local^T) + residual;
    backward: dx = all_gather(dy) @ W_local."""

    @staticmethod
    def forward(ctx, x, weight, residual, tp, impl):
        if impl == "fused":
            y = tp.gemm_rs(x, weight, residual=residual)
        else:
            y = tp.gemm_rs_nccl(x, weight, residual=residual)
        ctx.save_for_backward(x)
        ctx.wref, ctx.tp, ctx.impl, ctx.has_res = weight, tp, impl, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        (x,) = ctx.saved_tensors
        w, tp = ctx.wref, ctx.tp
        dy_shard = dy_shard.contiguous()
        # dx (M, K_loc) = all_gather(dy) (M,N) @ W (N, K_loc): B stored (K_c = N rows, K_loc)
        if ctx.impl == "fused":
            dx, dy_full = tp.ag_gemm(dy_shard, w, w_mn=True, keep_gathered=True)
        else:
            dx, dy_full = tp.ag_gemm_nccl(dy_shard, w, w_mn=True)
        mg = getattr(w, "main_grad", None)
        dres = dy_shard if ctx.has_res else None
        if mg is not None:
            gemm(dy_full, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
            w.grad_touched = True
            return dx, None, dres, None, None
        return dx, gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=w.dtype), dres, None, None


def column_parallel_linear(x_shard, weight, tp: TPContext, impl: str = "fused"):
    return _ColumnParallel.apply(x_shard, weight, tp, impl)


def row_parallel_linear(x, weight, tp: TPContext, residual=None, impl: str = "fused"):
    return _RowParallel.apply(x, weight, residual, tp, impl)
