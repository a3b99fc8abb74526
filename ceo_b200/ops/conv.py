"""Causal depthwise short convolution (``csrc/conv.cu``): y[t,d] = sum_w x[t-w,d] W[d,w].
Reference: src/model/prism.zig:448-476 (CPU loop); the CUDA entry point is declared only
(kernels/cuda/include/kernels.h:107)."""
from __future__ import annotations

import torch

from . import _lib, reference as ref


class _ShortConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        B, T, D = x.shape
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _lib.check(_lib.lib().ceo_shortconv_fwd(xc.data_ptr(), weight.data_ptr(), y.data_ptr(), B,
                                                T, D, weight.shape[1], _lib.stream()),
                   "ceo_shortconv_fwd")
        ctx.save_for_backward(xc, weight)
        ctx.wref = weight
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, _ = ctx.saved_tensors
        weight = ctx.wref
        B, T, D = xc.shape
        Wn = weight.shape[1]
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        L = _lib.lib()
        _lib.check(L.ceo_shortconv_bwd_input(dyc.data_ptr(), weight.data_ptr(), dx.data_ptr(), B,
                                             T, D, Wn, _lib.stream()), "ceo_shortconv_bwd_input")
        mg = getattr(weight, "main_grad", None)
        if mg is not None:
            buf, acc, ret = mg, 1, None
            weight.grad_touched = True
        else:
            buf = torch.empty(D, Wn, dtype=torch.float32, device=xc.device)
            acc, ret = 0, buf
        _lib.check(L.ceo_shortconv_bwd_weight(dyc.data_ptr(), xc.data_ptr(), buf.data_ptr(), B, T,
                                              D, Wn, acc, _lib.stream()),
                   "ceo_shortconv_bwd_weight")
        return dx, (ret.to(weight.dtype) if ret is not None else None)


def shortconv(x, weight):
    """x: (B,T,D) bf16; weight: (D, window)."""
    if not x.is_cuda:
        return ref.shortconv(x, weight)
    return _ShortConvFn.apply(x, weight)
