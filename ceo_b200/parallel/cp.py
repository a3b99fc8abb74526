"""Context parallelism for EFLA: the sequence is split over the ranks of a group and the
recurrent state crosses rank boundaries as an affine map.

Over one rank's span the delta-rule recurrence is ``S_out = P_r S_in + R_r`` with
``P_r = prod_c (I - K_c^T W_c)`` (so is its adjoint: ``dS_in = P_r^T dS_out + Q_r``).  Forward:

  A. every rank, in parallel: W, U of its chunks; R_r (state pass from zero) and P_r (state
     pass on the identity with U = 0);
  X. ``ceo_cp_exchange``: each rank stores (P_r, R_r) into every peer's gather buffer over
     NVLink and joins a flag barrier, in one kernel; every rank then folds the maps of the
     ranks before it into its true incoming state (G-1 tiny fp32 matmuls per head);
  B. the real state pass from that state, and the output kernel.

Backward mirrors it with Q_r and the transposed maps, folding from the last rank down.
The reference has only the flag ``use_ring_attention`` and an additive "chunked scan" stub
(src/tensor/sharding.zig:229, kernels/cuda/efla.cu:711-748, src/model/efla.zig:473-484).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib, efla as efla_ops
from .symm import SymmetricBuffer

_IDX = {"q": 0, "k": 1, "v": 2, "alpha": 3, "w": 4, "u": 5, "up": 6, "states": 7, "o": 8,
        "s0": 9, "s_final": 10, "dO": 11, "dloc": 12, "dup": 13, "dstates": 14, "ds_final": 15,
        "ds0": 16, "dq": 17, "dk": 18, "dv": 19, "dalpha": 20, "p_final": 21, "xinv": 23, "resets": 24}


def _stage(stage: int, tensors: dict, strides, B, T, H, d):
    ptrs = (ctypes.c_void_p * 25)()
    for k, t in tensors.items():
        ptrs[_IDX[k]] = None if t is None else t.data_ptr()
    ptrs[22] = _lib.status_word(torch.device("cuda", torch.cuda.current_device())).data_ptr()
    st = (ctypes.c_longlong * 6)(*strides)
    _lib.check(_lib.lib().ceo_efla_stage(stage, ptrs, st, B, T, H, d, _lib.stream()),
               f"ceo_efla_stage({stage})")


class CPContext:
    """Exchange buffers of one context-parallel group for up to ``max_bh`` (batch x heads)
    states of size d x d."""

    def __init__(self, comm, max_bh: int, d: int):
        self.comm, self.rank, self.world = comm, comm.rank, comm.world
        self.d, self.max_bh = d, max_bh
        self.slot_floats = 2 * max_bh * d * d
        # two gather areas used alternately: the kernel's own barrier says every rank has
        # STORED its block of this call, which (stream order) it only does after it has consumed
        # the call before - so when a rank writes an area again, two calls later, nobody reads
        # it any more.  No barrier before the exchange, no copy of the result.
        self.half_bytes = self.world * self.slot_floats * 4
        self.gather = SymmetricBuffer(2 * self.half_bytes, comm.group)
        self.calls = 0
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.done = torch.zeros(1, dtype=torch.int32, device=self.dev)

    def exchange(self, block: torch.Tensor) -> torch.Tensor:
        """block: fp32 tensor (same numel on every rank).  Returns (world, *block.shape): slot s
        = rank s's block - a view of the gather area, valid until the exchange after the next
        one (consume it, or copy what must live longer)."""
        n = block.numel()
        assert n % 4 == 0 and n <= self.slot_floats and block.dtype == torch.float32
        block = block.contiguous()
        self.calls += 1
        off = (self.calls & 1) * self.half_bytes
        L = _lib.lib()
        _lib.check(L.ceo_cp_exchange(block.data_ptr(), self.gather.table(off),
                                     self.comm.ctrl.table(), n, self.rank, self.world,
                                     self.comm._next_epoch(), self.done.data_ptr(),
                                     _lib.status_word(self.dev).data_ptr(), _lib.stream()),
                   "ceo_cp_exchange")
        return self.gather.view(torch.float32, self.world * n, off).view(self.world, *block.shape)

    def close(self):
        self.gather.close()


def fold_affine(P, s, R, transpose: bool = False):
    """``P s + R`` (or ``P^T s + R``) for batches of d x d fp32 matrices: one step of
    composing a rank's affine state map onto a state.  Runs on the library's own fp32 kernel
    (``ceo_fold_affine``); the first step of a fold (s = 0) just returns R."""
    if not P.is_cuda:
        return torch.matmul(P.transpose(-1, -2) if transpose else P, s) + R
    d = P.shape[-1]
    nb = P.numel() // (d * d)
    P, s, R = P.contiguous(), s.contiguous(), R.contiguous()
    out = torch.empty_like(s)
    _lib.check(_lib.lib().ceo_fold_affine(P.data_ptr(), s.data_ptr(), R.data_ptr(), out.data_ptr(),
                                          nb, d, int(transpose), _lib.stream()), "ceo_fold_affine")
    return out


class _CPDeltaRule(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, alpha, cp):
        B, T, H, d = k.shape
        n = T // efla_ops.CHUNK
        dev = k.device
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        alpha = alpha.contiguous().float()
        hd = H * d
        strides = (hd, hd, hd, hd, hd, hd)
        new = lambda: torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        w, u, up, o = new(), new(), new(), new()
        states = torch.empty(B, H, n, d, d, dtype=torch.bfloat16, device=dev)
        xinv = torch.empty(B, H, n, efla_ops.CHUNK, efla_ops.CHUNK, dtype=torch.bfloat16,
                           device=dev)
        R = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        P = torch.empty_like(R)
        base = {"q": q, "k": k, "v": v, "alpha": alpha, "w": w, "u": u, "up": up,
                "states": states, "o": o, "xinv": xinv}
        _stage(0, base, strides, B, T, H, d)
        # one launch: R_r (state pass from zero) and P_r (homogeneous pass on the identity)
        _stage(1, dict(base, s0=None, s_final=R, p_final=P), strides, B, T, H, d)
        allmaps = cp.exchange(torch.stack([P, R]))          # (G, 2, B, H, d, d)
        s_in = torch.zeros_like(R)
        for j in range(cp.rank):                            # fold the maps of earlier ranks
            s_in = fold_affine(allmaps[j, 0], s_in, allmaps[j, 1])
        s_out = torch.empty_like(R)
        _stage(1, dict(base, s0=s_in, s_final=s_out), strides, B, T, H, d)
        _stage(2, base, strides, B, T, H, d)
        ctx.save_for_backward(q, k, v, alpha, w, up, states, xinv, allmaps[:, 0].contiguous())
        ctx.cp = cp
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, alpha, w, up, states, xinv, Pall = ctx.saved_tensors
        cp = ctx.cp
        B, T, H, d = k.shape
        n = T // efla_ops.CHUNK
        dev = k.device
        hd = H * d
        strides = (hd, hd, hd, hd, hd, hd)
        do = do.contiguous()
        new = lambda: torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        dq, dk, dv, dloc, dup = new(), new(), new(), new(), new()
        dstates = torch.empty_like(states)
        dalpha = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        Q = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        base = {"q": q, "k": k, "v": v, "alpha": alpha, "w": w, "up": up, "states": states,
                "xinv": xinv, "dO": do, "dloc": dloc, "dup": dup, "dstates": dstates, "dq": dq, "dk": dk,
                "dv": dv, "dalpha": dalpha}
        _stage(3, base, strides, B, T, H, d)
        _stage(4, dict(base, ds_final=None, ds0=Q), strides, B, T, H, d)   # Q_r
        allq = cp.exchange(Q)                                              # (G, B, H, d, d)
        ds_out = torch.zeros_like(Q)
        for j in range(cp.world - 1, cp.rank, -1):                          # fold from the end
            ds_out = fold_affine(Pall[j], ds_out, allq[j], transpose=True)
        ds0 = torch.empty_like(Q)
        _stage(4, dict(base, ds_final=ds_out, ds0=ds0), strides, B, T, H, d)
        _stage(5, base, strides, B, T, H, d)
        return dq, dk, dv, dalpha, None


def cp_delta_rule(q, k, v, alpha, cp: CPContext):
    """Delta-rule attention over a sequence split across ``cp``'s ranks (rank r holds the r-th
    contiguous span).  q, k, v: (B, T_local, H, d) bf16; alpha: (B, T_local, H)."""
    return _CPDeltaRule.apply(q, k, v, alpha, cp)


def efla_flops(B, T, H, d, backward: bool = True) -> float:
    """Matmul FLOPs of the chunked kernels per call (forward, plus backward when asked)."""
    C = efla_ops.CHUNK
    per_chunk_fwd = 2 * (C * C * d            # K K^T
                         + 2 * C * C * d      # W, U
                         + 2 * C * d * d      # W S, K^T U'
                         + C * C * d          # Q K^T
                         + C * d * d          # Q S
                         + C * C * d)         # P U'
    per_chunk_bwd = 2 * (4 * C * C * d + 4 * C * d * d + 5 * C * C * d   # final
                         + 2 * C * C * d + C * d * d + 2 * C * C * d     # local
                         + 3 * C * d * d)                                # state bwd
    chunks = B * H * (T // C)
    return chunks * (per_chunk_fwd + (per_chunk_bwd if backward else 0))
