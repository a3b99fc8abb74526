"""Collectives fused with compute over peer-mapped memory (``csrc/comm.cu``).

``FusedComm`` keeps the ``Comm`` interface (NCCL stays available for rare or odd-shaped
collectives and as the measured baseline) and adds:

* ``alloc``: symmetric allocation for the flat parameter / gradient buffers,
* ``zero_step``: ONE cooperative kernel per rank doing gradient reduce-scatter (peer loads),
  global-norm clipping, AdamW or Lion on the rank's fp32 master shard, the bf16 parameter
  all-gather (peer stores) and gradient zeroing,
* ``bucket_reduce``: the reduce-scatter of one bucket of parameters on a side stream, so it
  overlaps the rest of the backward pass (ZeRO stage 2 and 3),
* ``barrier`` / ``all_reduce_small`` on device flags.

Launch requirement: every rank launches its kernel on its own GPU (one process per GPU);
the kernels wait for each other through bounded polls on flag words.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _lib
from .comm import Comm
from .symm import SymmetricBuffer


class FusedComm(Comm):
    fused = True

    def __init__(self, group=None):
        super().__init__(group)
        if self.world > 8:
            raise ValueError("peer-memory collectives support at most 8 ranks (one NVSwitch box)")
        if not torch.cuda.is_available():
            raise RuntimeError("FusedComm needs CUDA")
        self.dev = torch.device("cuda", torch.cuda.current_device())
        # control block: 8 flag slots x 8 ranks (u32) | 8 floats norm slots | 64 floats all-reduce
        self.ctrl = SymmetricBuffer(4096, group)
        self.epoch = 2
        self._buffers = [self.ctrl]
        self._local_acc = torch.zeros(2, dtype=torch.float32, device=self.dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=self.dev)

    # ---- allocation ---------------------------------------------------------------------
    def alloc(self, numel: int, dtype: torch.dtype):
        """Returns (local tensor, SymmetricBuffer) of ``numel`` elements, zero-filled."""
        nb = numel * torch.empty((), dtype=dtype).element_size()
        buf = SymmetricBuffer(nb, self.group)
        self._buffers.append(buf)
        return buf.view(dtype, numel), buf

    def _next_epoch(self) -> int:
        self.epoch += 2
        return self.epoch

    # ---- device-side barrier / small all-reduce -------------------------------------------
    def device_barrier(self):
        L = _lib.lib()
        _lib.check(L.ceo_symm_barrier(self.ctrl.table(), self.rank, self.world, 3,
                                      self._next_epoch(), _lib.status_word(self.dev).data_ptr(),
                                      _lib.stream()), "ceo_symm_barrier")

    def all_reduce_small(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of a small fp32 vector (<= 64 elements) across ranks, in one kernel."""
        n = t.numel()
        assert t.dtype == torch.float32 and n <= 64
        stage = self.ctrl.view(torch.float32, 64, 1024)
        stage[:n].copy_(t.reshape(-1))
        L = _lib.lib()
        out = torch.empty_like(t)
        _lib.check(L.ceo_symm_allreduce(self.ctrl.table(1024), self.ctrl.table(), out.data_ptr(), n,
                                        self.rank, self.world, self._next_epoch(),
                                        _lib.status_word(self.dev).data_ptr(), _lib.stream()),
                   "ceo_symm_allreduce")
        return out

    # ---- the fused optimizer step -----------------------------------------------------------
    def zero_step(self, flat, m, v, *, lr, betas, eps, weight_decay, step, grad_scale, max_norm,
                  kind: str = "adamw", do_reduce: bool = True, clip_out=None, max_ctas: int = 0):
        """Reduce-scatter (unless the bucket reductions already ran) + clip + AdamW / Lion +
        all-gather + zero-grad for a ``FlatParams`` whose parameter and gradient buffers came
        from ``alloc``.  Returns the gradient norm (device); ``clip_out`` (1 float, device)
        receives the clip scale, 0 when the step was skipped for a non-finite norm."""
        L = _lib.lib()
        rg = flat.ranges_device()
        _lib.check(L.ceo_zero_step(
            flat.grads_symm.table(), flat.params_symm.table(), self.ctrl.table(),
            self.ctrl.table(512), flat.master.data_ptr(), m.data_ptr(), _lib.ptr(v),
            self._local_acc.data_ptr(), self._norm.data_ptr(), _lib.ptr(clip_out),
            _lib.status_word(self.dev).data_ptr(), rg.data_ptr(), rg.shape[0], flat.total,
            flat.decay_end, self.rank, self.world, self._next_epoch(),
            {"adamw": 0, "lion": 1}[kind], int(do_reduce), float(lr), betas[0],
            betas[1], eps, weight_decay, step, float(grad_scale), float(max_norm), int(max_ctas),
            _lib.stream()), "ceo_zero_step")
        return self._norm

    def bucket_reduce(self, flat, r0: int, r1: int, stream, ctas: int = 24):
        """Flag barrier + reduce-scatter of ownership ranges [r0, r1) of ``flat`` on
        ``stream`` (a side stream that already waits for the bucket's last gradient kernel).
        Every rank must call this for the same buckets in the same order."""
        L = _lib.lib()
        rg = flat.ranges_device()
        _lib.check(L.ceo_zero_bucket_reduce(
            flat.grads_symm.table(), self.ctrl.table(), rg.data_ptr(), r0, r1, self.rank,
            self.world, self._next_epoch(), self._local_acc.data_ptr(),
            _lib.status_word(self.dev).data_ptr(), ctas, stream.cuda_stream),
            "ceo_zero_bucket_reduce")

    def close(self):
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self._buffers:
            b.close()
        self._buffers = []
