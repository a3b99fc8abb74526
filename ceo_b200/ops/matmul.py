"""bf16 GEMM on tcgen05/TMEM (``csrc/gemm_tcgen05.cu``) and the autograd Linear on top of it.

Layout vocabulary: the kernel computes ``C[M,N] = alpha * A[M,K] @ B[N,K]^T`` and
each operand may be stored K-major (rows of K) or MN-major (rows of M or N), so
forward, data-gradient and weight-gradient all read their tensors in place with
no transpose copy.  Weights are kept ``(out_features, in_features)``; the
reference stores ``(in, out)`` (src/nn/layers.zig:509,529) - the checkpoint
writer transposes.

The weight gradient can be accumulated straight into an fp32 ``main_grad``
buffer by the GEMM epilogue, which is how micro-batch gradient accumulation is
done without a separate add kernel.  Replaces gemm_forward_cuda /
gemm_backward_cuda of the reference (kernels/cuda/gemm.cu:303, 400).
"""
from __future__ import annotations

import os

import torch

from . import _lib


def _as2d(t: torch.Tensor) -> torch.Tensor:
    return t if t.dim() == 2 else t.reshape(-1, t.shape[-1])


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
         accumulate: bool = False, alpha: float = 1.0, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, max_ctas: int = 0) -> torch.Tensor:
    """``out = alpha * A @ B^T (+ bias) (+ residual) (+ out if accumulate)``.

    ``a`` is ``(M, K)`` (or ``(K, M)`` when ``a_mn``); ``b`` is ``(N, K)`` (or ``(K, N)``
    when ``b_mn``).  A leading batch dimension on both makes it a batched GEMM.
    """
    batched = a.dim() == 3
    if batched:
        assert b.dim() == 3 and a.shape[0] == b.shape[0]
        nb = a.shape[0]
        a2, b2 = a[0], b[0]
    else:
        nb = 1
        a2, b2 = a, b
    if a_mn:
        K, M = a2.shape
    else:
        M, K = a2.shape
    if b_mn:
        Kb, N = b2.shape
    else:
        N, Kb = b2.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"

    if not a.is_cuda:  # fp32 oracle path
        af = a.float().transpose(-1, -2) if a_mn else a.float()
        bf = b.float() if b_mn else b.float().transpose(-1, -2)
        r = alpha * (af @ bf)
        if bias is not None:
            r = r + bias.float()
        if residual is not None:
            r = r + residual.float()
        if out is not None:
            if accumulate:
                r = r + out.float()
            out.copy_(r.to(out.dtype))
            return out
        return r.to(out_dtype or a.dtype)

    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a2.stride(-1) == 1 and b2.stride(-1) == 1, "operands must have a unit inner stride"
    if out is None:
        shape = (nb, M, N) if batched else (M, N)
        out = torch.empty(shape, dtype=out_dtype or torch.bfloat16, device=a.device)
        assert not accumulate
    assert out.stride(-1) == 1
    out_f32 = out.dtype == torch.float32
    assert out_f32 or out.dtype == torch.bfloat16
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.stride(-1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous()
    rc = _lib.lib().ceo_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
        a2.stride(0), b2.stride(0), out.stride(-2), int(a_mn), int(b_mn), nb,
        a.stride(0) if batched else 0, b.stride(0) if batched else 0,
        out.stride(0) if batched else 0, int(out_f32), int(accumulate), float(alpha),
        _lib.ptr(bias), _lib.ptr(residual),
        residual.stride(-2) if residual is not None else 0,
        residual.stride(0) if (residual is not None and batched) else 0,
        _lib.status_word(a.device).data_ptr(), int(max_ctas), _lib.stream())
    _lib.check(rc, "ceo_gemm_bf16")
    return out


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ residual); dW accumulated into ``weight.main_grad`` when present."""

    @staticmethod
    def forward(ctx, x, weight, residual):
        x2 = _as2d(x)
        res2 = _as2d(residual) if residual is not None else None
        fg = getattr(weight, "fsdp_gather", None)
        if fg is not None and fg.pending:
            # FSDP: the weight is still row shards; its all-gather rides inside this GEMM
            y = fg.gemm(x2 if x2.is_contiguous() else x2.contiguous(), res2)
        else:
            y = gemm(x2, weight, residual=res2)
        ctx.save_for_backward(x2, weight)
        ctx.weight_ref = weight  # the Parameter object itself (carries .main_grad)
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, _ = ctx.saved_tensors
        weight = ctx.weight_ref
        dy2 = _as2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(weight, "main_grad", None)
            if mg is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
                weight.grad_touched = True
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        dres = dy if ctx.has_res else None
        return dx, dw, dres


def linear(x: torch.Tensor, weight: torch.Tensor,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ residual)`` with ``weight`` of shape ``(out, in)``."""
    return _LinearFn.apply(x, weight, residual)


# ---------------------------------------------------------------- SwiGLU MLP, fused
# False (or CEO_FUSED_SWIGLU=0 in the environment) runs the MLP as three separate ops
# (gate/up GEMM, SwiGLU kernel, down GEMM).
FUSED_SWIGLU = os.environ.get("CEO_FUSED_SWIGLU", "1") not in ("0", "")


def _gemm_swiglu(a, b, c, M, N, K, b_mn, mode, aux):
    rc = _lib.lib().ceo_gemm_bf16_swiglu(
        a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0), c.stride(0),
        0, int(b_mn), 1.0, mode, aux.data_ptr(), aux.stride(0),
        _lib.status_word(a.device).data_ptr(), _lib.stream())
    _lib.check(rc, "ceo_gemm_bf16_swiglu")


class _SwiGLUMlpFn(torch.autograd.Function):
    """``(silu(gate) * up) @ w_down^T (+ residual)`` with ``[gate, up] = x @ w_up^T`` in
    interleaved columns (row 2j of ``w_up`` is gate_j, row 2j+1 is up_j).

    Forward: the gate/up GEMM applies SiLU(gate) * up in its epilogue and writes gate/up (kept
    for the backward pass) and the activation together - no separate activation kernel, no
    re-read of gate/up.  Backward: the down projection's data-gradient GEMM reads gate/up in
    its epilogue and writes d(gate/up) directly; d(activation) never goes to memory."""

    @staticmethod
    def forward(ctx, x, w_up, w_down, residual):
        x2 = _as2d(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M, K = x2.shape
        N2 = w_up.shape[0]
        F = N2 // 2
        res2 = _as2d(residual) if residual is not None else None
        fg = getattr(w_up, "fsdp_gather", None)
        act = torch.empty(M, F, dtype=x2.dtype, device=x2.device)
        if fg is not None and fg.pending:
            # FSDP: this GEMM carries the weight all-gather; the activation runs on its own
            gate_up = fg.gemm(x2)
            _lib.check(_lib.lib().ceo_swiglu_il_fwd(gate_up.data_ptr(), act.data_ptr(), M, F, 1,
                                                    _lib.stream()), "ceo_swiglu_il_fwd")
        else:
            gate_up = torch.empty(M, N2, dtype=x2.dtype, device=x2.device)
            _gemm_swiglu(x2, w_up, gate_up, M, N2, K, False, 1, act)
        y = gemm(act, w_down, residual=res2)
        ctx.save_for_backward(x2, gate_up, act)
        ctx.refs = (w_up, w_down)
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, gate_up, act = ctx.saved_tensors
        w_up, w_down = ctx.refs
        M, K = x2.shape
        N2 = w_up.shape[0]
        F = N2 // 2
        D = w_down.shape[0]
        dy2 = _as2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # d(gate/up) from the down projection's data gradient: (M, D) x (D, F) -> epilogue
        dgu = torch.empty_like(gate_up)
        _gemm_swiglu(dy2, w_down, dgu, M, F, D, True, 2, gate_up)
        grads = []
        for w, dyy, xin in ((w_down, dy2, act), (w_up, dgu, x2)):
            mg = getattr(w, "main_grad", None)
            if not w.requires_grad:
                grads.append(None)
            elif mg is not None:
                gemm(dyy, xin, a_mn=True, b_mn=True, out=mg, accumulate=True)
                w.grad_touched = True
                grads.append(None)
            else:
                grads.append(gemm(dyy, xin, a_mn=True, b_mn=True, out_dtype=w.dtype))
        dx = gemm(dgu, w_up, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        return dx, grads[1], grads[0], (dy if ctx.has_res else None)


def swiglu_mlp(x, w_up, w_down, residual=None):
    """The SwiGLU MLP ``(silu(x W_gate^T) * (x W_up^T)) W_down^T (+ residual)`` with the
    activation fused into the GEMM epilogues; ``w_up`` holds gate and up rows interleaved."""
    return _SwiGLUMlpFn.apply(x, w_up, w_down, residual)
