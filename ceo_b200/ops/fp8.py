"""FP8 training path: per-tensor delayed scaling, the tcgen05 ``kind::f8f6f4`` GEMM and a
Linear whose forward product runs on e4m3 operands.

The reference only names this feature: a ``fp8_training`` switch (src/util/config.zig:420,
configs/train.yaml:56), an ``enable-fp8`` build option (build.zig:18), the ``ScaleFactor``
delayed-scaling record (src/tensor/dtype.zig:85-128) and header-only quantise / dequantise
entry points (kernels/cuda/kernels.h:378-395); no GEMM of its ever sees an 8-bit operand.

Recipe here: activations and weights are quantised to e4m3 with one scale per tensor,
``q = sat(x * scale)``, where the scale comes from the largest magnitude seen over the last 16
steps (``Fp8Meta``).  ``y = (q_x q_w^T) / (scale_x scale_w)`` is formed by the GEMM epilogue,
which reads both scales from device memory, so no step of the recipe synchronises with the
host.  By default the data- and weight-gradient products stay in bf16 (they read the saved
bf16 activation and the bf16 weight), which keeps the gradients those of the bf16 model
evaluated at an fp8-perturbed forward.  With ``Fp8Recipe(dgrad=True)`` the data gradient
``dx = dy W`` also runs on 8-bit operands: dy in e5m2 (its own delayed scale) against an e4m3
copy of ``W^T``, so that both operands are K-major.  With ``wgrad=True`` the weight gradient
``dW = dy^T x`` does too: one kernel writes the codes of a tensor and of its transpose from a
single read, the forward keeps ``q(x)^T`` (one byte per element) for the backward instead of
the bf16 activation, and the GEMM accumulates into the fp32 gradient buffer as the bf16 one
does.  Quantised weights (and their transposes) are cached for the whole optimizer step.

Without a GPU the same arithmetic runs through ``torch.float8_e4m3fn`` casts in fp32.
"""
from __future__ import annotations

import torch

from . import _lib
from .matmul import _as2d, gemm, linear
from .tensor_ops import transpose2d

E4M3, E5M2 = 0, 1
_FMAX = {E4M3: 448.0, E5M2: 57344.0}
_TORCH = {E4M3: torch.float8_e4m3fn, E5M2: torch.float8_e5m2}


class Fp8Meta:
    """Delayed-scaling state of one tensor, all of it on the tensor's device: current scale,
    running amax of the step in progress, amax history ring and its cursor."""

    def __init__(self, device, kind: int = E4M3, history: int = 16, margin: int = 0):
        self.kind, self.margin, self.device = kind, margin, torch.device(device)
        self.scale = torch.ones(1, dtype=torch.float32, device=device)
        self.amax = torch.zeros(1, dtype=torch.float32, device=device)
        self.history = torch.zeros(history, dtype=torch.float32, device=device)
        self.cursor = torch.zeros(1, dtype=torch.int32, device=device)
        self.calibrated = False

    def update(self) -> None:
        """Push the step's amax into the history and derive the next scale from its maximum."""
        if self.device.type == "cuda":
            _lib.check(_lib.lib().ceo_fp8_update_scale(
                self.history.data_ptr(), self.history.numel(), self.cursor.data_ptr(),
                self.amax.data_ptr(), self.scale.data_ptr(), _FMAX[self.kind],
                float(2.0 ** self.margin), _lib.stream()), "ceo_fp8_update_scale")
        else:
            n = self.history.numel()
            self.history[int(self.cursor) % n] = self.amax[0]
            self.cursor[0] = (int(self.cursor) + 1) % n
            m = float(self.history.max())
            ok = m > 0 and m == m and m != float("inf")
            self.scale[0] = _FMAX[self.kind] / (m * 2.0 ** self.margin) if ok else 1.0
            self.amax.zero_()
        self.calibrated = True

    def state_dict(self) -> dict:
        return {"scale": float(self.scale), "cursor": int(self.cursor),
                "history": [float(v) for v in self.history.tolist()],
                "calibrated": bool(self.calibrated)}

    def load_state_dict(self, d: dict) -> None:
        self.scale.fill_(float(d["scale"]))
        self.cursor.fill_(int(d["cursor"]))
        self.history.copy_(torch.tensor(d["history"], dtype=torch.float32))
        self.amax.zero_()
        self.calibrated = bool(d["calibrated"])


def quantize(x: torch.Tensor, meta: Fp8Meta) -> torch.Tensor:
    """``sat(x * meta.scale)`` as raw 8-bit codes (uint8, same shape); ``meta.amax`` takes the
    maximum with ``max |x|``.  A tensor seen for the first time is measured first, so that even
    the first step uses a scale that fits it."""
    x = x.contiguous()
    if not meta.calibrated:
        _quantize_raw(x, meta)
        meta.update()
    return _quantize_raw(x, meta)


def _quantize_raw(x: torch.Tensor, meta: Fp8Meta) -> torch.Tensor:
    if not x.is_cuda:
        xf = x.float()
        meta.amax.copy_(torch.maximum(meta.amax, xf.abs().max().reshape(1)))
        lim = _FMAX[meta.kind]
        return (xf * meta.scale).clamp(-lim, lim).to(_TORCH[meta.kind]).view(torch.uint8)
    assert x.dtype == torch.bfloat16
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib().ceo_fp8_quantize(x.data_ptr(), q.data_ptr(), x.numel(),
                                           meta.scale.data_ptr(), meta.amax.data_ptr(),
                                           meta.kind, _lib.stream()), "ceo_fp8_quantize")
    return q


def quantize_t(x: torch.Tensor, meta: Fp8Meta, want_q: bool = True):
    """Codes of the 2-D tensor ``x`` and of its transpose from one read: ``(q or None, qt)``
    with ``q`` of shape (rows, cols) and ``qt`` of shape (cols, rows)."""
    assert x.dim() == 2
    x = x.contiguous()
    if not meta.calibrated:
        _quantize_raw(x, meta)
        meta.update()
    rows, cols = x.shape
    if not x.is_cuda or rows % 16 or cols % 16:
        q = _quantize_raw(x, meta)
        return (q if want_q else None), q.t().contiguous()
    assert x.dtype == torch.bfloat16
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device) if want_q else None
    qt = torch.empty(cols, rows, dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib().ceo_fp8_quantize_t(x.data_ptr(), _lib.ptr(q), qt.data_ptr(), rows, cols,
                                             x.stride(0), meta.scale.data_ptr(),
                                             meta.amax.data_ptr(), meta.kind, _lib.stream()),
               "ceo_fp8_quantize_t")
    return q, qt


def gemm_fp8(aq: torch.Tensor, bq: torch.Tensor, a_meta: Fp8Meta | None = None,
             b_meta: Fp8Meta | None = None, *, kind_a: int | None = None,
             kind_b: int | None = None, out: torch.Tensor | None = None,
             out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
             alpha: float = 1.0, bias: torch.Tensor | None = None,
             residual: torch.Tensor | None = None) -> torch.Tensor:
    """``out = alpha / (scale_a scale_b) * A @ B^T (+ bias) (+ residual) (+ out if accumulate)``
    with ``aq`` (M, K) and ``bq`` (N, K) holding 8-bit float codes (uint8).  The metas give the
    element formats and the scales to undo; without them the codes are multiplied as they are.
    """
    assert aq.dtype == torch.uint8 and bq.dtype == torch.uint8 and aq.dim() == 2 and bq.dim() == 2
    M, K = aq.shape
    N, Kb = bq.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    assert (a_meta is None) == (b_meta is None)
    ka = a_meta.kind if a_meta is not None else (kind_a or E4M3)
    kb = b_meta.kind if b_meta is not None else (kind_b or E4M3)
    if not aq.is_cuda:
        r = alpha * (aq.view(_TORCH[ka]).float() @ bq.view(_TORCH[kb]).float().t())
        if a_meta is not None:
            r = r / (a_meta.scale * b_meta.scale)
        if bias is not None:
            r = r + bias.float()
        if residual is not None:
            r = r + residual.float()
        if out is not None:
            if accumulate:
                r = r + out.float()
            out.copy_(r.to(out.dtype))
            return out
        return r.to(out_dtype)
    assert aq.stride(1) == 1 and bq.stride(1) == 1
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=out_dtype, device=aq.device)
    assert out.stride(-1) == 1 and out.dtype in (torch.float32, torch.bfloat16)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.stride(-1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous()
    rc = _lib.lib().ceo_gemm_fp8(
        aq.data_ptr(), bq.data_ptr(), out.data_ptr(), M, N, K, aq.stride(0), bq.stride(0),
        out.stride(0), ka, kb, int(out.dtype == torch.float32), int(accumulate), float(alpha),
        _lib.ptr(a_meta.scale) if a_meta is not None else None,
        _lib.ptr(b_meta.scale) if b_meta is not None else None,
        _lib.ptr(bias), _lib.ptr(residual),
        residual.stride(0) if residual is not None else 0,
        _lib.status_word(aq.device).data_ptr(), _lib.stream())
    _lib.check(rc, "ceo_gemm_fp8")
    return out


class Fp8LinearState:
    """What one Linear keeps between calls: the metas of its input and weight and the weight's
    quantised copy, valid for one optimizer step (``Fp8Recipe.step`` invalidates it)."""

    def __init__(self, device, recipe: "Fp8Recipe"):
        self.x_meta = Fp8Meta(device, E4M3, recipe.history, recipe.margin)
        self.w_meta = Fp8Meta(device, E4M3, recipe.history, recipe.margin)
        self.g_meta = Fp8Meta(device, E5M2, recipe.history, recipe.margin)
        self.wq = None
        self.wq_step = -1
        self.wtq = None
        self.wtq_step = -1
        self.recipe = recipe

    def weight_q(self, weight: torch.Tensor) -> torch.Tensor:
        if self.wq is None or self.wq_step != self.recipe.step_id:
            self.wq = quantize(weight.detach(), self.w_meta)
            self.wq_step = self.recipe.step_id
        return self.wq

    def weight_t_q(self, weight: torch.Tensor) -> torch.Tensor:
        """e4m3 codes of ``weight^T`` (in, out), on the scale of ``weight_q``."""
        if self.wtq is None or self.wtq_step != self.recipe.step_id:
            self.weight_q(weight)  # makes sure the weight's scale is calibrated
            self.wtq = _quantize_raw(transpose2d(weight.detach()), self.w_meta)
            self.wtq_step = self.recipe.step_id
        return self.wtq


class Fp8Recipe:
    """Owner of every ``Fp8LinearState`` of a model; ``step()`` is called once per optimizer
    step, after the parameters changed."""

    def __init__(self, history: int = 16, margin: int = 0, dgrad: bool = False,
                 wgrad: bool = False):
        self.history, self.margin, self.dgrad, self.wgrad = history, margin, dgrad, wgrad
        self.states: list[Fp8LinearState] = []
        self.step_id = 0

    def new_state(self, device) -> Fp8LinearState:
        st = Fp8LinearState(device, self)
        self.states.append(st)
        return st

    def step(self) -> None:
        for st in self.states:
            if st.x_meta.calibrated:
                st.x_meta.update()
            if st.w_meta.calibrated:
                st.w_meta.update()
            if st.g_meta.calibrated:
                st.g_meta.update()
        self.step_id += 1

    def invalidate(self) -> None:
        """Drops the cached weight codes (call after the parameters were replaced, e.g. by a
        checkpoint load, outside an optimizer step)."""
        for st in self.states:
            st.wq = st.wtq = None

    def state_dict(self) -> dict:
        """Scales and amax histories of every tensor (plain numbers: goes into a checkpoint's
        metadata); cached weight codes are rebuilt on the next use."""
        return {"history": self.history, "margin": self.margin,
                "states": [[m.state_dict() for m in (st.x_meta, st.w_meta, st.g_meta)]
                           for st in self.states]}

    def load_state_dict(self, d: dict) -> None:
        if len(d["states"]) != len(self.states) or d["history"] != self.history:
            raise ValueError("FP8 state of a different model or recipe")
        for st, ms in zip(self.states, d["states"]):
            for m, md in zip((st.x_meta, st.w_meta, st.g_meta), ms):
                m.load_state_dict(md)
        self.invalidate()


class _Fp8LinearFn(torch.autograd.Function):
    """y = dequant(q(x) q(W)^T) (+ residual); gradients as in the bf16 Linear, or on 8-bit
    operands where the recipe says so."""

    @staticmethod
    def forward(ctx, x, weight, residual, state):
        x2 = _as2d(x)
        rec = state.recipe
        fp8_w = rec.wgrad and x2.shape[0] % 16 == 0 and x2.shape[1] % 16 == 0 \
            and weight.shape[0] % 16 == 0
        if fp8_w:
            xq, xqt = quantize_t(x2, state.x_meta)
        else:
            xq, xqt = quantize(x2, state.x_meta), None
        wq = state.weight_q(weight)
        y = gemm_fp8(xq, wq, state.x_meta, state.w_meta, out_dtype=x.dtype,
                     residual=_as2d(residual) if residual is not None else None)
        ctx.save_for_backward(xqt if fp8_w else x2, weight)
        ctx.fp8_w = fp8_w
        ctx.weight_ref = weight
        ctx.state = state
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xs, _ = ctx.saved_tensors
        weight = ctx.weight_ref
        state = ctx.state
        rec = state.recipe
        dy2 = _as2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        fp8_d = rec.dgrad and need_x and weight.shape[0] % 16 == 0
        fp8_w = ctx.fp8_w and need_w
        dyq = dyqt = None
        if fp8_w:
            dyq, dyqt = quantize_t(dy2, state.g_meta, want_q=fp8_d)
        elif fp8_d:
            dyq = quantize(dy2, state.g_meta)
        dx = None
        if need_x:
            if fp8_d:
                dx = gemm_fp8(dyq, state.weight_t_q(weight), state.g_meta, state.w_meta,
                              out_dtype=dy.dtype).view(ctx.x_shape)
            else:
                dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        dw = None
        if need_w:
            mg = getattr(weight, "main_grad", None)
            if fp8_w:
                if mg is not None:
                    gemm_fp8(dyqt, xs, state.g_meta, state.x_meta, out=mg, accumulate=True)
                else:
                    dw = gemm_fp8(dyqt, xs, state.g_meta, state.x_meta, out_dtype=weight.dtype)
            elif mg is not None:
                gemm(dy2, xs, a_mn=True, b_mn=True, out=mg, accumulate=True)
            else:
                dw = gemm(dy2, xs, a_mn=True, b_mn=True, out_dtype=weight.dtype)
            if mg is not None:
                weight.grad_touched = True
        return dx, dw, (dy if ctx.has_res else None), None


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, state: Fp8LinearState,
               residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ residual)`` with the product taken on e4m3 operands (rows of 8-bit
    operands must be multiples of 16 bytes: other widths take the bf16 Linear)."""
    if x.shape[-1] % 16:
        return linear(x, weight, residual)
    return _Fp8LinearFn.apply(x, weight, residual, state)
