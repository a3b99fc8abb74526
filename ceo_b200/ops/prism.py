"""PRISM refinement ops (``csrc/prism.cu``): the fused gate of one iteration with its
backward, the fused residual / output update, and the recurrent state.  CPU tensors run the
fp32 PyTorch form of the same math.

Reference: the layer's specification in src/model/prism.zig:11-40, ``PrismState`` 480-523; the
CUDA entry point ``prism_forward_cuda`` is declared only (kernels/cuda/include/kernels.h:86).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


def gate_reference(rp, p, bt):
    """bd = sigmoid(bt) * GELU_tanh(p * rp) in fp32."""
    return torch.sigmoid(bt.float()) * F.gelu(p.float() * rp.float(), approximate="tanh")


class _GateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rp, p, bt):
        rp, p, bt = rp.contiguous(), p.contiguous(), bt.contiguous()
        bd = torch.empty_like(rp)
        _lib.check(_lib.lib().ceo_prism_gate_fwd(rp.data_ptr(), p.data_ptr(), bt.data_ptr(),
                                                 bd.data_ptr(), rp.numel(), _lib.stream()),
                   "ceo_prism_gate_fwd")
        ctx.save_for_backward(rp, p, bt)
        return bd

    @staticmethod
    def backward(ctx, dbd):
        rp, p, bt = ctx.saved_tensors
        dbd = dbd.contiguous()
        drp, dp, dbt = torch.empty_like(rp), torch.empty_like(p), torch.empty_like(bt)
        _lib.check(_lib.lib().ceo_prism_gate_bwd(dbd.data_ptr(), rp.data_ptr(), p.data_ptr(),
                                                 bt.data_ptr(), drp.data_ptr(), dp.data_ptr(),
                                                 dbt.data_ptr(), rp.numel(), _lib.stream()),
                   "ceo_prism_gate_bwd")
        return drp, dp, dbt


def gate(rp, p, bt):
    """``sigmoid(bt) * GELU(p * rp)`` for (.., hd) bf16 tensors (one kernel each way)."""
    if not rp.is_cuda or rp.dtype != torch.bfloat16 or rp.numel() % 8:
        return gate_reference(rp, p, bt).to(rp.dtype)
    return _GateFn.apply(rp, p, bt)


class _UpdateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, c, r, out, scale):
        c, r, out = c.contiguous(), r.contiguous(), out.contiguous()
        r2, o2 = torch.empty_like(r), torch.empty_like(out)
        _lib.check(_lib.lib().ceo_prism_update(c.data_ptr(), r.data_ptr(), out.data_ptr(),
                                               r2.data_ptr(), o2.data_ptr(), c.numel(),
                                               float(scale), _lib.stream()), "ceo_prism_update")
        ctx.scale = scale
        return r2, o2

    @staticmethod
    def backward(ctx, dr, do):
        dc = None
        if dr is not None and do is not None:
            dc = do * ctx.scale - dr
        elif do is not None:
            dc = do * ctx.scale
        elif dr is not None:
            dc = -dr
        return dc, dr, do, None


def update(c, r, out, scale: float):
    """``(r - c, out + scale * c)`` in one pass over the streams."""
    if not c.is_cuda or c.dtype != torch.bfloat16 or c.numel() % 8:
        return r - c, out + scale * c
    return _UpdateFn.apply(c, r, out, scale)


def state_reference(bd, k, bt1, s_in, alpha: float):
    """Token-serial fp32 recurrence.  bd, k: (L, B, T, hd); bt1: (B, T, hd); s_in: (B, hd, hd)
    or None.  Returns S_T (B, hd, hd)."""
    L, B, T, hd = bd.shape
    s = torch.zeros(B, hd, hd, dtype=torch.float32, device=bd.device) if s_in is None \
        else s_in.float().clone()
    bdf, kf = bd.float(), k.float()
    b = torch.sigmoid(bt1.float()) * kf[0]
    for t in range(T):
        sb = torch.einsum("bij,bj->bi", s, b[:, t])
        s = alpha * (s - sb[:, :, None] * kf[0, :, t][:, None, :])
        for l in range(L):
            s = s + bdf[l, :, t][:, :, None] * kf[l, :, t][:, None, :]
    return s


@torch.no_grad()
def state(bd, k, bt1, s_in, alpha: float):
    """The PRISM state after the T tokens of ``bd`` / ``k`` (see ``state_reference``)."""
    L, B, T, hd = bd.shape
    if not bd.is_cuda or hd not in (32, 64, 128) or L > 4:
        return state_reference(bd, k, bt1, s_in, alpha)
    bd, k, bt1 = (t.to(torch.bfloat16).contiguous() for t in (bd, k, bt1))
    out = torch.empty(B, hd, hd, dtype=torch.float32, device=bd.device)
    sin = None if s_in is None else s_in.float().contiguous()
    _lib.check(_lib.lib().ceo_prism_state(bd.data_ptr(), k.data_ptr(), bt1.data_ptr(),
                                          _lib.ptr(sin), out.data_ptr(), B, T, hd, L, float(alpha),
                                          _lib.stream()), "ceo_prism_state")
    return out
