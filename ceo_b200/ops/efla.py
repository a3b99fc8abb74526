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


def _tok_stride(t: torch.Tensor) -> int:
    """Row (token) stride in elements of a (B,T,H,d) tensor whose (H,d) block is dense and
    whose (B,T) dimensions collapse to one stride (true for slices of a fused QKV output)."""
    B, T, H, d = t.shape
    assert t.stride(3) == 1 and t.stride(2) == d, "head block must be dense"
    assert B == 1 or t.stride(0) == T * t.stride(1), "(B,T) must collapse"
    return t.stride(1)


class _DeltaRuleFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, alpha, s0):
        B, T, H, d = k.shape
        assert v.shape[-1] == d and d in (64, 128), "head_dim must be 64 or 128"
        assert T % CHUNK == 0, "sequence length must be a multiple of 64"
        n = T // CHUNK
        dev = k.device
        alpha = alpha.contiguous().float()
        w = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        up = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        o = torch.empty(B, T, H, d, dtype=torch.bfloat16, device=dev)
        states = torch.empty(B, H, n, d, d, dtype=torch.bfloat16, device=dev)
        s_final = torch.empty(B, H, d, d, dtype=torch.float32, device=dev)
        L = _lib.lib()
        st = _lib.status_word(dev).data_ptr()
        _lib.check(L.ceo_efla_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), alpha.data_ptr(),
                                  _lib.ptr(s0), w.data_ptr(), up.data_ptr(), states.data_ptr(),
                                  o.data_ptr(), s_final.data_ptr(), B, T, H, d, _tok_stride(q),
                                  _tok_stride(k), _tok_stride(v), st, _lib.stream()),
                   "ceo_efla_fwd")
        ctx.save_for_backward(q, k, v, alpha, w, up, states)
        ctx.has_s0 = s0 is not None
        return o, s_final

    @staticmethod
    def backward(ctx, do, ds_final):
        q, k, v, alpha, w, up, states = ctx.saved_tensors
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
                                  w.data_ptr(), up.data_ptr(), states.data_ptr(), do.data_ptr(),
                                  _lib.ptr(ds_final), dloc.data_ptr(), dup.data_ptr(),
                                  dstates.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                  dalpha.data_ptr(), ds0.data_ptr(), B, T, H, d, _tok_stride(q),
                                  _tok_stride(k), _tok_stride(v), st, _lib.stream()),
                   "ceo_efla_bwd")
        return dq, dk, dv, dalpha, (ds0 if ctx.has_s0 else None)


def delta_rule(q, k, v, alpha, s0=None, impl: str = "auto"):
    """Delta-rule linear attention.  q,k,v: (B,T,H,d) bf16; alpha: (B,T,H).
    Returns ``(o, S_T)`` with ``S_T`` the fp32 final state (B,H,d,d).

    ``impl``: "auto" (CUDA kernels on GPU, chunked oracle on CPU), "chunked" or
    "sequential" (fp32 PyTorch oracles, any device)."""
    if impl == "sequential":
        o, s = ref.delta_rule_sequential(q, k, v, alpha, s0)
        return o.to(q.dtype), s
    if impl == "chunked" or not k.is_cuda:
        T = k.shape[1]
        pad = (-T) % CHUNK
        if pad:  # zero-alpha padding tokens leave the state untouched
            zp = lambda t: torch.nn.functional.pad(t, (0, 0, 0, 0, 0, pad))
            o, s = ref.delta_rule_chunked(zp(q), zp(k), zp(v),
                                          torch.nn.functional.pad(alpha, (0, 0, 0, pad)), s0,
                                          CHUNK)
            return o[:, :T].to(q.dtype), s
        o, s = ref.delta_rule_chunked(q, k, v, alpha, s0, CHUNK)
        return o.to(q.dtype), s
    return _DeltaRuleFn.apply(q, k, v, alpha, s0)


def l2norm(x, eps: float = 1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def efla_attention(q, k, v, beta, *, normalize_qk: bool = True, s0=None, impl: str = "auto"):
    """q,k,v: (B,T,H,d); beta: (B,T,H) (already positive, e.g. a sigmoid) or a scalar tensor.
    Returns (o, S_T)."""
    if normalize_qk:
        q = l2norm(q)
        k = l2norm(k)
    lam = k.float().pow(2).sum(-1)
    alpha = ref.efla_coefficient(beta.float().expand_as(lam), lam)
    return delta_rule(q, k, v, alpha, s0, impl)


def delta_rule_decode_step(q, k, v, alpha, state):
    """One recurrent token step for generation.  q,k,v: (B,H,d); alpha: (B,H);
    state: (B,H,d,d) fp32, updated in place.  Returns o: (B,H,d)."""
    kf, vf, qf = k.float(), v.float(), q.float()
    u = torch.einsum("bhkv,bhk->bhv", state, kf)
    state.add_(alpha.float()[..., None, None] * torch.einsum("bhk,bhv->bhkv", kf, vf - u))
    return torch.einsum("bhkv,bhk->bhv", state, qf).to(q.dtype)
