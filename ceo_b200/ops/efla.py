"""EFLA attention: exact-solution delta-rule linear attention.

    lambda_t = ||k_t||^2        alpha_t = (1 - exp(-beta_t * lambda_t)) / lambda_t
    S_t = (I - alpha_t k_t k_t^T) S_{t-1} + alpha_t k_t v_t^T        o_t = S_t^T q_t

``delta_rule`` is the core (per-token step ``alpha``); on CUDA it runs the chunked
kernels of ``csrc/efla.cu`` (WY/UT transform per 64-token chunk on tensor cores, fp32
inter-chunk state, backward recomputed from per-chunk states).  ``efla_attention`` adds
the optional L2 normalisation of q/k and the coefficient.  The reference's kernel is the
special case q = k with one scalar beta and walks the sequence token by token
(kernels/cuda/efla.cu:154-233; backward 315-454 stores every S_t).
"""
from __future__ import annotations

import torch

from . import _lib, reference as ref

CHUNK = 64


def _resets_u8(resets, B: int, n: int, dev):
    """(B, T/64) mask -> contiguous uint8 on the device (None stays None)."""
    if resets is None:
        return None
    r = resets.to(device=dev, dtype=torch.uint8).contiguous()
    assert r.shape == (B, n), "resets must have shape (B, T/64)"
    return r


def _tok_stride(t: torch.Tensor) -> int:
    """Row (token) stride in elements of a (B,T,H,d) tensor whose (H,d) block is dense and
    whose (B,T) dimensions collapse to one stride (true for slices of a fused QKV output)."""
    B, T, H, d = t.shape
    assert t.stride(3) == 1 and t.stride(2) == d, "head block must be dense"
    assert B == 1 or t.stride(0) == T * t.stride(1), "(B,T) must collapse"
    return t.stride(1)


class _DeltaRuleFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, alpha, s0, resets=None):
        B, T, H, d = k.shape
        assert v.shape[-1] == d and d in (64, 128), "head_dim must be 64 or 128"
        assert T % CHUNK == 0, "sequence length must be a multiple of 64"
        n = T // CHUNK
        dev = k.device
        ctx.resets = resets = _resets_u8(resets, B, n, dev)
        alpha = alpha.contiguous().float()
        w = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        up = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        o = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        states = torch.empty(B, H, n, d, d, dtype=torch.bfloat16, device=dev)
        xinv = torch.empty(B, H, n, CHUNK, CHUNK, dtype=torch.bfloat16, device=dev)
        s_final = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        L = _lib.lib()
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), alpha.data_ptr(),
                                  _lib.ptr(s0), w.data_ptr(), up.data_ptr(), states.data_ptr(),
                                  xinv.data_ptr(),
                                  o.data_ptr(), s_final.data_ptr(), _lib.ptr(resets), B, T, H, d,
                                  _tok_stride(q), _tok_stride(k), _tok_stride(v), st,
                                  _lib.stream()),
                   "ceo_efla_fwd")
        ctx.save_for_backward(q, k, v, alpha, w, up, states, xinv)
        ctx.has_s0 = s0 is not None
        return o, s_final

    @staticmethod
    def backward(ctx, do, ds_final):
        q, k, v, alpha, w, up, states, xinv = ctx.saved_tensors
        B, T, H, d = k.shape
        n = T // CHUNK
        dev = k.device
        do = do.contiguous()
        dq = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        dk = torch.empty_like(dq)
        dv = torch.empty_like(dq)
        dalpha = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        dloc = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        dup = torch.empty_like(dloc)
        dstates = torch.empty(B, H, n, d, d, dtype=torch.bfloat16, device=dev)
        ds0 = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        if ds_final is not None:
            ds_final = ds_final.contiguous().float()
        L = _lib.lib()
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), alpha.data_ptr(),
                                  w.data_ptr(), up.data_ptr(), states.data_ptr(), xinv.data_ptr(),
                                  do.data_ptr(),
                                  _lib.ptr(ds_final), dloc.data_ptr(), dup.data_ptr(),
                                  dstates.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                  dalpha.data_ptr(), ds0.data_ptr(), _lib.ptr(ctx.resets), B, T, H, d,
                                  _tok_stride(q), _tok_stride(k), _tok_stride(v), H * d, H * d,
                                  H * d, st, _lib.stream()),
                   "ceo_efla_bwd")
        return dq, dk, dv, dalpha, (ds0 if ctx.has_s0 else None), None


class _EflaQKVFn(torch.autograd.Function):
    """EFLA attention straight off a fused projection output ``qkv`` of shape
    (B, T, P, H, d) with P = 3 (q, k, v) or P = 2 (k, v; q = k as in the reference).
    One kernel normalises q/k and computes alpha; the chunked kernels follow; backward
    writes dq, dk, dv into one (B, T, P, H, d) buffer so the projection's gradient GEMMs
    read it in place."""

    @staticmethod
    def forward(ctx, qkv, beta, normalize, s0, resets=None):
        B, T, P, H, d = qkv.shape
        assert qkv.is_contiguous() and P in (2, 3) and T % CHUNK == 0
        dev = qkv.device
        n = T // CHUNK
        ctx.resets = resets = _resets_u8(resets, B, n, dev)
        ts = P * H * d
        q_raw = qkv[:, :, 0] if P == 3 else qkv[:, :, 0]
        k_raw = qkv[:, :, 1] if P == 3 else qkv[:, :, 0]
        v = qkv[:, :, P - 1]
        beta = beta.float().contiguous()
        scalar = beta.numel() == 1
        rows = B * T
        L = _lib.lib()
        qn = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        kn = torch.empty_like(qn) if P == 3 else qn
        rq = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        rk = torch.empty_like(rq)
        alpha = torch.empty_like(rq)
        _lib.check(L.ceo_efla_prep_fwd(q_raw.data_ptr(), k_raw.data_ptr(), beta.data_ptr(),
                                       int(scalar), qn.data_ptr(), kn.data_ptr(), rq.data_ptr(),
                                       rk.data_ptr(), alpha.data_ptr(), rows, H, d, ts, ts,
                                       int(normalize), _lib.stream()), "ceo_efla_prep_fwd")
        w = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        up = torch.empty_like(w)
        o = torch.empty_like(w)
        states = torch.empty(B, H, n, d, d, dtype=torch.bfloat16, device=dev)
        xinv = torch.empty(B, H, n, CHUNK, CHUNK, dtype=torch.bfloat16, device=dev)
        s_final = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_fwd(qn.data_ptr(), kn.data_ptr(), v.data_ptr(), alpha.data_ptr(),
                                  _lib.ptr(s0), w.data_ptr(), up.data_ptr(), states.data_ptr(),
                                  xinv.data_ptr(),
                                  o.data_ptr(), s_final.data_ptr(), _lib.ptr(resets), B, T, H, d,
                                  H * d, H * d, ts,
                                  st, _lib.stream()), "ceo_efla_fwd")
        ctx.save_for_backward(qkv, beta, qn, kn, rq, rk, alpha, w, up, states, xinv)
        ctx.cfg = (normalize, scalar, s0 is not None)
        return o, s_final

    @staticmethod
    def backward(ctx, do, ds_final):
        qkv, beta, qn, kn, rq, rk, alpha, w, up, states, xinv = ctx.saved_tensors
        normalize, scalar, has_s0 = ctx.cfg
        B, T, P, H, d = qkv.shape
        n = T // CHUNK
        dev = qkv.device
        ts = P * H * d
        do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        dqn = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        dkn = torch.empty_like(dqn)
        dalpha = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        dloc = torch.empty_like(dqn)
        dup = torch.empty_like(dqn)
        dstates = torch.empty_like(states)
        ds0 = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        if ds_final is not None:
            ds_final = ds_final.contiguous().float()
        v = qkv[:, :, P - 1]
        dv = dqkv[:, :, P - 1]
        L = _lib.lib()
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_bwd(qn.data_ptr(), kn.data_ptr(), v.data_ptr(), alpha.data_ptr(),
                                  w.data_ptr(), up.data_ptr(), states.data_ptr(), xinv.data_ptr(),
                                  do.data_ptr(),
                                  _lib.ptr(ds_final), dloc.data_ptr(), dup.data_ptr(),
                                  dstates.data_ptr(), dqn.data_ptr(), dkn.data_ptr(),
                                  dv.data_ptr(), dalpha.data_ptr(), ds0.data_ptr(),
                                  _lib.ptr(ctx.resets), B, T, H, d,
                                  H * d, H * d, ts, H * d, H * d, ts, st, _lib.stream()),
                   "ceo_efla_bwd")
        dbeta = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        if P == 3:
            dq_out, dk_out = dqkv[:, :, 0], dqkv[:, :, 1]
        else:  # q = k: both gradients land on the one projection
            dkn.add_(dqn)
            dq_out = dloc  # scratch: the q-side output of the kernel is unused
            dk_out = dqkv[:, :, 0]
        _lib.check(L.ceo_efla_prep_bwd(dqn.data_ptr(), dkn.data_ptr(), qn.data_ptr(),
                                       kn.data_ptr(), rq.data_ptr(), rk.data_ptr(),
                                       beta.data_ptr(), int(scalar), dalpha.data_ptr(),
                                       dq_out.data_ptr(), dk_out.data_ptr(), dbeta.data_ptr(),
                                       B * T, H, d, (ts if P == 3 else H * d), ts,
                                       int(normalize), _lib.stream()), "ceo_efla_prep_bwd")
        if scalar:
            dbeta = dbeta.sum().reshape(beta.shape)
        return dqkv, dbeta, None, (ds0 if has_s0 else None), None


def efla_qkv(qkv, beta, normalize: bool = True, s0=None, resets=None):
    """EFLA attention on a fused projection output.  qkv: (B,T,P,H,d), P = 3 (q,k,v) or 2
    (k,v with q = k); beta: (B,T,H) or a one-element tensor.  Returns (o (B,T,H,d), S_T)."""
    if not qkv.is_cuda:
        P = qkv.shape[2]
        q = qkv[:, :, 0]
        k = qkv[:, :, 1] if P == 3 else qkv[:, :, 0]
        return efla_attention(q, k, qkv[:, :, P - 1], beta, normalize_qk=normalize, s0=s0,
                              resets=resets)
    return _EflaQKVFn.apply(qkv, beta, normalize, s0, resets)


def delta_rule(q, k, v, alpha, s0=None, impl: str = "auto", resets=None):
    """Delta-rule linear attention.  q,k,v: (B,T,H,d) bf16; alpha: (B,T,H).
    Returns ``(o, S_T)`` with ``S_T`` the fp32 final state (B,H,d,d).

    ``resets``: optional (B, T/64) mask; a set entry means that 64-token chunk starts a new
    document, so the state entering it is zero (packed sequences aligned to the chunk).

    ``impl``: "auto" (CUDA kernels on GPU, chunked oracle on CPU), "chunked" or
    "sequential" (fp32 PyTorch oracles, any device)."""
    if impl == "sequential":
        o, s = ref.delta_rule_sequential(q, k, v, alpha, s0, resets, CHUNK)
        return o.to(q.dtype), s
    if impl == "chunked" or not k.is_cuda:
        T = k.shape[1]
        pad = (-T) % CHUNK
        if pad:  # zero-alpha padding tokens leave the state untouched
            assert resets is None, "resets need a sequence length that is a multiple of 64"
            zp = lambda t: torch.nn.functional.pad(t, (0, 0, 0, 0, 0, pad))
            o, s = ref.delta_rule_chunked(zp(q), zp(k), zp(v),
                                          torch.nn.functional.pad(alpha, (0, 0, 0, pad)), s0,
                                          CHUNK)
            return o[:, :T].to(q.dtype), s
        o, s = ref.delta_rule_chunked(q, k, v, alpha, s0, CHUNK, resets)
        return o.to(q.dtype), s
    return _DeltaRuleFn.apply(q, k, v, alpha, s0, resets)


def l2norm(x, eps: float = 1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def efla_attention(q, k, v, beta, *, normalize_qk: bool = True, s0=None, impl: str = "auto",
                   resets=None):
    """q,k,v: (B,T,H,d); beta: (B,T,H) (already positive, e.g. a sigmoid) or a scalar tensor.
    Returns (o, S_T)."""
    if normalize_qk:
        q = l2norm(q)
        k = l2norm(k)
    lam = k.float().pow(2).sum(-1)
    alpha = ref.efla_coefficient(beta.float().expand_as(lam), lam)
    return delta_rule(q, k, v, alpha, s0, impl, resets)


def delta_rule_decode_step(q, k, v, alpha, state):
    """One recurrent token step for generation.  q,k,v: (B,H,d); alpha: (B,H);
    state: (B,H,d,d) fp32, updated in place.  Returns o: (B,H,d)."""
    kf, vf, qf = k.float(), v.float(), q.float()
    u = torch.einsum("bhkv,bhk->bhv", state, kf)
    state.add_(alpha.float()[..., None, None] * torch.einsum("bhk,bhv->bhkv", kf, vf - u))
    return torch.einsum("bhkv,bhk->bhv", state, qf).to(q.dtype)


class _EflaProjFn(torch.autograd.Function):
    """EFLA attention straight off ONE projection output ``proj`` (B, T, N) whose columns are
    ``[q (H*d) | k (H*d) | v (H*d) | beta logits (H) | padding]`` (no q block when P = 2).
    The per-token beta = sigmoid(logit) is taken from the same buffer, and backward fills one
    (B, T, N) gradient buffer in place - q/k/v slices by the kernels, the logit columns from
    d(beta) - so the projection's gradient GEMMs read it without any concatenation."""

    @staticmethod
    def forward(ctx, proj, P, H, d, normalize, s0, resets=None):
        B, T, N = proj.shape
        assert proj.is_contiguous() and N >= P * H * d + H and N % 8 == 0 and T % CHUNK == 0
        dev = proj.device
        n = T // CHUNK
        ctx.resets = resets = _resets_u8(resets, B, n, dev)
        hd = H * d
        esz = proj.element_size()
        base = proj.data_ptr()
        q_ptr, k_ptr = base, base + (hd * esz if P == 3 else 0)
        v_ptr = base + (P - 1) * hd * esz
        beta = torch.sigmoid(proj[..., P * hd:P * hd + H].float()).contiguous()
        L = _lib.lib()
        qn = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        kn = torch.empty_like(qn) if P == 3 else qn
        rq = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        rk = torch.empty_like(rq)
        alpha = torch.empty_like(rq)
        _lib.check(L.ceo_efla_prep_fwd(q_ptr, k_ptr, beta.data_ptr(), 0, qn.data_ptr(),
                                       kn.data_ptr(), rq.data_ptr(), rk.data_ptr(),
                                       alpha.data_ptr(), B * T, H, d, N, N, int(normalize),
                                       _lib.stream()), "ceo_efla_prep_fwd")
        w = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        up = torch.empty_like(w)
        o = torch.empty_like(w)
        states = torch.empty(B, H, n, d, d, dtype=torch.bfloat16, device=dev)
        xinv = torch.empty(B, H, n, CHUNK, CHUNK, dtype=torch.bfloat16, device=dev)
        s_final = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_fwd(qn.data_ptr(), kn.data_ptr(), v_ptr, alpha.data_ptr(),
                                  _lib.ptr(s0), w.data_ptr(), up.data_ptr(), states.data_ptr(),
                                  xinv.data_ptr(),
                                  o.data_ptr(), s_final.data_ptr(), _lib.ptr(resets), B, T, H, d,
                                  hd, hd, N, st,
                                  _lib.stream()), "ceo_efla_fwd")
        ctx.save_for_backward(proj, beta, qn, kn, rq, rk, alpha, w, up, states, xinv)
        ctx.cfg = (P, H, d, normalize, s0 is not None)
        return o, s_final

    @staticmethod
    def backward(ctx, do, ds_final):
        proj, beta, qn, kn, rq, rk, alpha, w, up, states, xinv = ctx.saved_tensors
        P, H, d, normalize, has_s0 = ctx.cfg
        B, T, N = proj.shape
        dev = proj.device
        hd = H * d
        esz = proj.element_size()
        do = do.contiguous()
        dproj = torch.empty_like(proj)
        dqn = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        dkn = torch.empty_like(dqn)
        dalpha = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        dloc = torch.empty_like(dqn)
        dup = torch.empty_like(dqn)
        dstates = torch.empty_like(states)
        ds0 = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        if ds_final is not None:
            ds_final = ds_final.contiguous().float()
        base, dbase = proj.data_ptr(), dproj.data_ptr()
        v_ptr, dv_ptr = base + (P - 1) * hd * esz, dbase + (P - 1) * hd * esz
        L = _lib.lib()
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_bwd(qn.data_ptr(), kn.data_ptr(), v_ptr, alpha.data_ptr(),
                                  w.data_ptr(), up.data_ptr(), states.data_ptr(), xinv.data_ptr(),
                                  do.data_ptr(),
                                  _lib.ptr(ds_final), dloc.data_ptr(), dup.data_ptr(),
                                  dstates.data_ptr(), dqn.data_ptr(), dkn.data_ptr(), dv_ptr,
                                  dalpha.data_ptr(), ds0.data_ptr(), _lib.ptr(ctx.resets), B, T, H,
                                  d, hd, hd, N, hd, hd,
                                  N, st, _lib.stream()), "ceo_efla_bwd")
        dbeta = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        if P == 3:
            dq_ptr, dk_ptr, dq_stride = dbase, dbase + hd * esz, N
        else:
            dkn.add_(dqn)
            dq_ptr, dk_ptr, dq_stride = dloc.data_ptr(), dbase, hd
        _lib.check(L.ceo_efla_prep_bwd(dqn.data_ptr(), dkn.data_ptr(), qn.data_ptr(),
                                       kn.data_ptr(), rq.data_ptr(), rk.data_ptr(),
                                       beta.data_ptr(), 0, dalpha.data_ptr(), dq_ptr, dk_ptr,
                                       dbeta.data_ptr(), B * T, H, d, dq_stride, N, int(normalize),
                                       _lib.stream()), "ceo_efla_prep_bwd")
        tail = dproj[..., P * hd:]
        tail.zero_()
        tail[..., :H].copy_(dbeta * beta * (1.0 - beta))
        return dproj, None, None, None, None, (ds0 if has_s0 else None), None


def efla_proj(proj, P: int, H: int, d: int, normalize: bool = True, s0=None, resets=None):
    """EFLA attention on a fused projection output with the beta logits in it.
    proj: (B, T, N), columns [q | k | v | H beta logits | pad] (P = 3) or [k | v | ...] (P = 2).
    Returns (o (B,T,H,d), S_T)."""
    if not proj.is_cuda:
        B, T, N = proj.shape
        hd = H * d
        qkv = proj[..., :P * hd].reshape(B, T, P, H, d)
        beta = torch.sigmoid(proj[..., P * hd:P * hd + H].float())
        q = qkv[:, :, 0]
        k = qkv[:, :, 1] if P == 3 else qkv[:, :, 0]
        return efla_attention(q, k, qkv[:, :, P - 1], beta, normalize_qk=normalize, s0=s0,
                              resets=resets)
    return _EflaProjFn.apply(proj, P, H, d, normalize, s0, resets)
