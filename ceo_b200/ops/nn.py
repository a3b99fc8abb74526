"""Autograd wrappers over the bandwidth-bound kernels: RMSNorm / LayerNorm (with the
pre-norm residual add folded in), SwiGLU / GELU / SiLU, embedding, softmax, and the
row-chunked LM-head + cross-entropy.  CPU tensors run the fp32 PyTorch oracle of the
same op (``ops/reference.py``); CUDA tensors always run the kernels.

Reference counterparts: src/nn/layers.zig:14-687 (CPU layers),
kernels/cuda/layernorm.cu:307-449 (kernels), src/kernels/nn_kernels.zig:111-248 (CPU refs).
"""
from __future__ import annotations

import torch

from . import _lib, reference as ref
from .matmul import gemm

ACT_MODES = {"gelu": 0, "gelu_tanh": 0, "gelu_erf": 1, "silu": 2, "relu": 3}


# --------------------------------------------------------------------------- RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps, skip=False):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        if residual is not None:
            r2 = residual.reshape(-1, D)
            h = torch.empty_like(x2)
        else:
            r2, h = None, None
        L = _lib.lib()
        _lib.check(L.ceo_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(r2), weight.data_ptr(), y.data_ptr(),
                                     _lib.ptr(h), rstd.data_ptr(), rows, D, float(eps),
                                     _lib.stream()), "ceo_rmsnorm_fwd")
        hin = h if h is not None else x2
        ctx.save_for_backward(hin, weight, rstd)
        ctx.weight_ref = weight
        ctx.shape = shp
        ctx.has_res = residual is not None
        if residual is not None:
            return y.view(shp), h.view(shp)
        if skip:
            # the input itself is the second output: the gradient of every other use of it (the
            # residual stream) arrives here as `dh` and is added inside the backward kernel
            return y.view(shp), x
        return y.view(shp), None

    @staticmethod
    def backward(ctx, dy, dh):
        hin, _, rstd = ctx.saved_tensors
        weight = ctx.weight_ref
        rows, D = hin.shape
        dy2 = dy.reshape(-1, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dh is not None:
            dres = dh.reshape(-1, D)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(hin)
        L = _lib.lib()
        nblk = L.ceo_norm_bwd_blocks(rows)
        scratch = _lib.scratch(hin.device, nblk * D, "norm")
        mg = getattr(weight, "main_grad", None)
        if mg is not None:
            dw_buf, acc, dw_ret = mg, 1, None
            weight.grad_touched = True
        else:
            dw_buf = torch.empty(D, dtype=torch.float32, device=hin.device)
            acc, dw_ret = 0, dw_buf
        _lib.check(L.ceo_rmsnorm_bwd(dy2.data_ptr(), hin.data_ptr(), weight.data_ptr(),
                                     rstd.data_ptr(), _lib.ptr(dres), dx.data_ptr(),
                                     dw_buf.data_ptr(), acc, scratch.data_ptr(), rows, D,
                                     _lib.stream()), "ceo_rmsnorm_bwd")
        dx = dx.view(ctx.shape)
        if dw_ret is not None:
            dw_ret = dw_ret.to(weight.dtype)
        return dx, dw_ret, (dx if ctx.has_res else None), None, None


def rmsnorm(x, weight, eps: float = 1e-6, residual=None, skip: bool = False):
    """``y = rmsnorm(x + residual) * weight``.  Returns ``(y, h)`` with ``h = x + residual``
    (``h`` is None when there is no residual).  ``skip=True`` (no residual): ``h`` is ``x``
    routed through this op, to be used wherever the residual stream continues, so that its
    gradient is added to the normalisation's inside the backward kernel instead of by a
    separate elementwise add."""
    if not x.is_cuda:
        y, h = ref.rmsnorm(x, weight, eps, residual)
        return y, (x if (skip and residual is None) else h)
    return _RMSNormFn.apply(x, weight, residual, eps, skip and residual is None)


# ------------------------------------------------------------------------- LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        L = _lib.lib()
        _lib.check(L.ceo_layernorm_fwd(x2.data_ptr(), weight.data_ptr(), _lib.ptr(bias),
                                       y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, D,
                                       float(eps), _lib.stream()), "ceo_layernorm_fwd")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.refs = (weight, bias)
        ctx.shape = shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, _, mean, rstd = ctx.saved_tensors
        weight, bias = ctx.refs
        rows, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dx = torch.empty_like(x2)
        L = _lib.lib()
        nblk = L.ceo_norm_bwd_blocks(rows)
        scratch = _lib.scratch(x2.device, nblk * 2 * D, "norm")
        mgw = getattr(weight, "main_grad", None)
        mgb = getattr(bias, "main_grad", None) if bias is not None else None
        use_main = mgw is not None and (bias is None or mgb is not None)
        if use_main:
            dw, db, acc = mgw, mgb, 1
            weight.grad_touched = True
            if bias is not None:
                bias.grad_touched = True
        else:
            dw = torch.empty(D, dtype=torch.float32, device=x2.device)
            db = torch.empty(D, dtype=torch.float32, device=x2.device) if bias is not None else None
            acc = 0
        _lib.check(L.ceo_layernorm_bwd(dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(),
                                       mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), _lib.ptr(db), acc, scratch.data_ptr(), rows,
                                       D, _lib.stream()), "ceo_layernorm_bwd")
        if use_main:
            return dx.view(ctx.shape), None, None, None
        return (dx.view(ctx.shape), dw.to(weight.dtype),
                db.to(bias.dtype) if bias is not None else None, None)


def layernorm(x, weight, bias=None, eps: float = 1e-5):
    if not x.is_cuda:
        return ref.layernorm(x, weight, bias, eps)
    return _LayerNormFn.apply(x, weight, bias, eps)


# ----------------------------------------------------------------------- activations
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up, interleaved):
        F = gate_up.shape[-1] // 2
        g2 = gate_up.reshape(-1, 2 * F)
        out = torch.empty(g2.shape[0], F, dtype=gate_up.dtype, device=gate_up.device)
        _lib.check(_lib.lib().ceo_swiglu_il_fwd(g2.data_ptr(), out.data_ptr(), g2.shape[0], F,
                                                int(interleaved), _lib.stream()),
                   "ceo_swiglu_il_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gate_up.shape
        ctx.interleaved = interleaved
        return out.view(*gate_up.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        F = g2.shape[-1] // 2
        d2 = dout.reshape(-1, F)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(g2)
        _lib.check(_lib.lib().ceo_swiglu_il_bwd(d2.data_ptr(), g2.data_ptr(), dgu.data_ptr(),
                                                g2.shape[0], F, int(ctx.interleaved),
                                                _lib.stream()), "ceo_swiglu_il_bwd")
        return dgu.view(ctx.shape), None


def swiglu(gate_up, interleaved: bool = False):
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dimension, or, with
    ``interleaved``, for gate and up in alternating columns (2j = gate_j, 2j+1 = up_j)."""
    if not gate_up.is_cuda:
        return ref.swiglu(gate_up, interleaved)
    assert gate_up.is_contiguous()
    return _SwiGLUFn.apply(gate_up, interleaved)


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mode):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _lib.check(_lib.lib().ceo_act_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), mode,
                                          _lib.stream()), "ceo_act_fwd")
        ctx.save_for_backward(xc)
        ctx.mode = mode
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        _lib.check(_lib.lib().ceo_act_bwd(dyc.data_ptr(), xc.data_ptr(), dx.data_ptr(),
                                          xc.numel(), ctx.mode, _lib.stream()), "ceo_act_bwd")
        return dx, None


def activation(x, kind: str = "gelu"):
    """Elementwise activation: gelu (tanh), gelu_erf, silu, relu."""
    if not x.is_cuda:
        return ref.activation(x, kind)
    return _ActFn.apply(x, ACT_MODES[kind])


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Softmax over dimension ``dim`` (fp32), as the reference's ``Softmax(dim)`` layer
    (src/nn/layers.zig:386-458).  The kernel reduces rows; another dimension is moved last."""
    if not x.is_cuda:
        return torch.softmax(x.float(), dim=dim)
    dim = dim % x.dim()
    if dim != x.dim() - 1:
        return softmax(x.movedim(dim, -1), -1).movedim(-1, dim)
    x2 = x.float().reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty_like(x2)
    _lib.check(_lib.lib().ceo_softmax_fwd(x2.data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1],
                                          _lib.stream()), "ceo_softmax_fwd")
    return y.view(x.shape)


# ---------------------------------------------------------------------------- dropout
def dropout_keep_mask(numel: int, p: float, seed: int, device="cpu") -> torch.Tensor:
    """The keep mask of ``ceo_dropout`` (the same integer hash in PyTorch): element i is kept
    iff the top 24 bits of hash(i, seed) are >= p * 2^24."""
    M = 0xFFFFFFFF
    idx = torch.arange(numel, dtype=torch.int64, device=device)
    x = ((idx & M) ^ (seed & M) ^ (((idx >> 32) * 0x9E3779B9) & M)) & M
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & M
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & M
    x = x ^ (x >> 16)
    return (x >> 8) >= int(p * 16777216.0)


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _lib.check(_lib.lib().ceo_dropout(xc.data_ptr(), y.data_ptr(), xc.numel(), float(p),
                                          int(seed) & 0xFFFFFFFF, _lib.stream()), "ceo_dropout")
        ctx.p, ctx.seed = p, seed
        return y

    @staticmethod
    def backward(ctx, dy):
        dyc = dy.contiguous()
        dx = torch.empty_like(dyc)
        _lib.check(_lib.lib().ceo_dropout(dyc.data_ptr(), dx.data_ptr(), dyc.numel(),
                                          float(ctx.p), int(ctx.seed) & 0xFFFFFFFF, _lib.stream()),
                   "ceo_dropout")
        return dx, None, None


_dropout_calls = [0]


def dropout(x: torch.Tensor, p: float, training: bool = True, seed: int | None = None):
    """Inverted dropout (reference: ``Dropout`` in src/nn/layers.zig:461-503; ``model.dropout``,
    src/util/config.zig:92,118).  The mask is a stateless hash of (element index, seed): nothing
    is stored for the backward pass.  ``seed`` defaults to the torch seed plus a call counter."""
    if not training or p <= 0.0:
        return x
    if not 0.0 <= p < 1.0:
        raise ValueError(f"dropout probability {p} is not in [0, 1)")
    if seed is None:
        _dropout_calls[0] += 1
        seed = (torch.initial_seed() * 0x9E3779B1 + _dropout_calls[0] * 0x85EBCA6B) & 0xFFFFFFFF
    if not x.is_cuda or x.dtype != torch.bfloat16:
        keep = dropout_keep_mask(x.numel(), p, seed, x.device).view(x.shape)
        return torch.where(keep, x / (1.0 - p), torch.zeros_like(x))
    return _DropoutFn.apply(x, p, seed)


# -------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        V, D = table.shape
        out = torch.empty(flat.numel(), D, dtype=table.dtype, device=table.device)
        _lib.check(_lib.lib().ceo_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(),
                                                flat.numel(), D, V, None, _lib.stream()),
                   "ceo_embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.table_ref = table
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        table = ctx.table_ref
        V, D = table.shape
        dy2 = dy.reshape(-1, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        mg = getattr(table, "main_grad", None)
        if mg is not None:
            buf, ret = mg, None
            table.grad_touched = True
        else:
            buf = torch.zeros(V, D, dtype=torch.float32, device=table.device)
            ret = buf
        _lib.check(_lib.lib().ceo_embedding_bwd(flat.data_ptr(), dy2.data_ptr(), buf.data_ptr(),
                                                flat.numel(), D, V, _lib.stream()),
                   "ceo_embedding_bwd")
        return None, (ret.to(table.dtype) if ret is not None else None)


def embedding(ids, table):
    if not table.is_cuda:
        return ref.embedding(ids, table)
    return _EmbeddingFn.apply(ids, table)


# ------------------------------------------------------------- LM head + cross-entropy
_pools = {}


def _workspace(device, nbytes: int):
    """The device's workspace pool (``utils.layout.MemoryPool``), grown when a call needs more."""
    from ..utils.layout import MemoryPool
    key = device.index if device.index is not None else torch.cuda.current_device()
    pool = _pools.get(key)
    if pool is None or pool.buf.numel() < nbytes:
        pool = MemoryPool(nbytes, device)
        _pools[key] = pool
    return pool


class _LinearCrossEntropyFn(torch.autograd.Function):
    """mean CE of ``x @ W^T`` against targets, row-chunked: logits exist only for one chunk
    at a time (fp32, from the GEMM epilogue); the CE kernel writes d(logits) in bf16 and the
    two gradient GEMMs of the chunk run before the next chunk's logits overwrite the buffer."""

    @staticmethod
    def forward(ctx, x, weight, targets, label_smoothing, ignore_index, chunk_rows):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        t = targets.reshape(-1).to(torch.int64).contiguous()
        rows, V = x2.shape[0], weight.shape[0]
        n_valid = (t != ignore_index).sum().clamp(min=1).to(torch.float32)
        inv = (1.0 / n_valid).reshape(1)
        losses = torch.empty(rows, dtype=torch.float32, device=x.device)
        need_grad = x.requires_grad or weight.requires_grad
        dx = torch.empty_like(x2) if need_grad else None
        mg = getattr(weight, "main_grad", None)
        dw = None
        if need_grad and mg is None:
            dw = torch.zeros(V, D, dtype=torch.float32, device=x.device)
        L = _lib.lib()
        cr = min(chunk_rows, rows)
        # logits and d(logits) of a chunk live in a step-scoped workspace pool (one buffer per
        # device, re-used by every call: both are dead when this function returns)
        pool = _workspace(x.device, cr * V * 6 + 1024)
        pool.reset()
        logits = pool.allocate((cr, V), torch.float32)
        dlog = pool.allocate((cr, V), torch.bfloat16) if need_grad else None
        for r0 in range(0, rows, cr):
            r1 = min(rows, r0 + cr)
            n = r1 - r0
            xc = x2[r0:r1]
            gemm(xc, weight, out=logits[:n])
            _lib.check(L.ceo_cross_entropy(logits.data_ptr(), 1, t[r0:r1].data_ptr(),
                                           losses[r0:r1].data_ptr(), _lib.ptr(dlog), n, V, V, V,
                                           float(label_smoothing), inv.data_ptr(), 1.0,
                                           int(ignore_index), _lib.stream()), "ceo_cross_entropy")
            if need_grad:
                gemm(dlog[:n], weight, b_mn=True, out=dx[r0:r1])
                gemm(dlog[:n], xc, a_mn=True, b_mn=True, out=mg if mg is not None else dw,
                     accumulate=True)
        if mg is not None and need_grad:
            weight.grad_touched = True
        loss = losses.sum() * inv[0]
        ctx.save_for_backward(dx, dw)
        ctx.x_shape = x.shape
        ctx.wdtype = weight.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        # gradients were computed with d(loss)=1; rescale if the caller scaled the loss
        gx = (dx * dloss.to(dx.dtype)).view(ctx.x_shape) if dx is not None else None
        gw = (dw * dloss).to(ctx.wdtype) if dw is not None else None
        return gx, gw, None, None, None, None


def linear_cross_entropy(x, weight, targets, label_smoothing: float = 0.0,
                         ignore_index: int = -100, chunk_rows: int = 16384):
    """Mean token cross-entropy of the LM head ``x @ weight.T`` without materialising the
    full logits.  With ``weight.main_grad`` set, dW is accumulated there during the forward
    pass assuming the loss is back-propagated with gradient 1 (the trainer folds its
    micro-batch scale into the optimizer's gradient scale instead)."""
    if not x.is_cuda:
        return ref.linear_cross_entropy(x, weight, targets, label_smoothing, ignore_index)
    return _LinearCrossEntropyFn.apply(x, weight, targets, label_smoothing, ignore_index,
                                       chunk_rows)


def cross_entropy_rows(logits, targets, label_smoothing: float = 0.0, ignore_index: int = -100):
    """Per-row CE losses (no gradient) - used by the evaluator."""
    if not logits.is_cuda:
        return ref.cross_entropy_rows(logits, targets, label_smoothing, ignore_index)
    l2 = logits.reshape(-1, logits.shape[-1])
    if l2.dtype not in (torch.float32, torch.bfloat16) or not l2.is_contiguous():
        l2 = l2.float().contiguous()
    t = targets.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty(l2.shape[0], dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().ceo_cross_entropy(l2.data_ptr(), int(l2.dtype == torch.float32),
                                            t.data_ptr(), out.data_ptr(), None, l2.shape[0],
                                            l2.shape[1], l2.stride(0), 0, float(label_smoothing),
                                            None, 1.0, int(ignore_index), _lib.stream()),
               "ceo_cross_entropy")
    return out
