"""fp32 PyTorch oracles for every kernel.  They are the CPU execution path of the ops,
the numerical reference of the GPU tests, and a restatement of the reference's math:

* EFLA recurrence: kernels/cuda/efla.cu:181-232 and src/kernels/efla_kernels.zig:49-108
* coefficient c(beta, lambda) with its small-lambda series: efla.cu:93-115
* RMSNorm / LayerNorm / softmax / cross-entropy: src/kernels/nn_kernels.zig:111-248
* Lion / AdamW / Newton-Schulz / clipping: src/kernels/optim_kernels.zig:79-218
* GELU: src/kernels/prism_kernels.zig:63-90;  ShortConv: src/model/prism.zig:448-476
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ norms / activations
def rmsnorm(x, weight, eps=1e-6, residual=None):
    h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype), (h if residual is not None else None)


def layernorm(x, weight, bias=None, eps=1e-5):
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps) * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def swiglu(gate_up, interleaved: bool = False):
    """silu(gate) * up; gate / up are the two halves of the last dimension, or (interleaved)
    its even / odd columns."""
    gf = gate_up.float()
    g, u = (gf[..., 0::2], gf[..., 1::2]) if interleaved else gf.chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def activation(x, kind="gelu"):
    xf = x.float()
    if kind in ("gelu", "gelu_tanh"):
        y = F.gelu(xf, approximate="tanh")
    elif kind == "gelu_erf":
        y = F.gelu(xf)
    elif kind == "silu":
        y = F.silu(xf)
    elif kind == "relu":
        y = F.relu(xf)
    else:
        raise ValueError(kind)
    return y.to(x.dtype)


def embedding(ids, table):
    return F.embedding(ids.long(), table)


def cross_entropy_rows(logits, targets, label_smoothing=0.0, ignore_index=-100):
    z = logits.float().reshape(-1, logits.shape[-1])
    t = targets.reshape(-1).long()
    lse = torch.logsumexp(z, dim=-1)
    tt = t.clamp(0, z.shape[-1] - 1)
    zt = z.gather(1, tt[:, None])[:, 0]
    loss = lse - (1.0 - label_smoothing) * zt - label_smoothing * z.mean(-1)
    valid = (t != ignore_index) & (t >= 0) & (t < z.shape[-1])
    return torch.where(valid, loss, torch.zeros_like(loss))


def linear_cross_entropy(x, weight, targets, label_smoothing=0.0, ignore_index=-100):
    logits = x.reshape(-1, x.shape[-1]).float() @ weight.float().t()
    t = targets.reshape(-1).long()
    rows = cross_entropy_rows(logits, t, label_smoothing, ignore_index)
    n = (t != ignore_index).sum().clamp(min=1)
    return rows.sum() / n


# ------------------------------------------------------------------------------- EFLA
def efla_coefficient(beta, lam):
    """c = (1 - exp(-beta*lam)) / lam, with the series beta - b^2 l/2 + b^3 l^2/6 - b^4 l^3/24
    for lam <= 1e-6."""
    small = lam <= 1e-6
    safe = torch.where(small, torch.ones_like(lam), lam)
    exact = -torch.expm1(-beta * safe) / safe
    series = beta - beta**2 * lam / 2 + beta**3 * lam**2 / 6 - beta**4 * lam**3 / 24
    return torch.where(small, series, exact)


def delta_rule_sequential(q, k, v, alpha, s0=None, resets=None, chunk=64):
    """Token-by-token delta rule.  q,k,v: (B,T,H,d); alpha: (B,T,H).
    S_t = (I - a_t k_t k_t^T) S_{t-1} + a_t k_t v_t^T ;  o_t = S_t^T q_t.
    ``resets`` (B, T/chunk): a set entry zeroes the state of that batch row before the first
    token of the chunk.  Returns (o (B,T,H,dv), S_T (B,H,dk,dv))."""
    B, T, H, dk = k.shape
    dv = v.shape[-1]
    qf, kf, vf, af = q.float(), k.float(), v.float(), alpha.float()
    S = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=k.device) if s0 is None \
        else s0.float().clone()
    outs = []
    for t in range(T):
        kt, vt, qt, at = kf[:, t], vf[:, t], qf[:, t], af[:, t]
        if resets is not None and t % chunk == 0:
            S = S * (~resets[:, t // chunk].bool()).to(S.dtype).view(B, 1, 1, 1)
        u = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + at[..., None, None] * torch.einsum("bhk,bhv->bhkv", kt, vt - u)
        outs.append(torch.einsum("bhkv,bhk->bhv", S, qt))
    return torch.stack(outs, dim=1), S


def delta_rule_chunked(q, k, v, alpha, s0=None, chunk=64, resets=None):
    """Chunkwise WY / UT-transform form of the same recurrence (what the CUDA kernels
    compute): per chunk A = strict_tril(diag(a) K K^T), T = (I+A)^-1 diag(a), W = T K,
    U = T V, U' = U - W S, O = Q S + tril(Q K^T) U', S += K^T U'."""
    B, T, H, dk = k.shape
    dv = v.shape[-1]
    assert T % chunk == 0
    n = T // chunk
    f = lambda x: x.float().view(B, n, chunk, H, -1).permute(0, 3, 1, 2, 4)  # B,H,n,C,d
    qf, kf, vf = f(q), f(k), f(v)
    af = alpha.float().view(B, n, chunk, H).permute(0, 3, 1, 2)  # B,H,n,C
    G = kf @ kf.transpose(-1, -2)
    A = torch.tril(af[..., None] * G, diagonal=-1)
    eye = torch.eye(chunk, device=k.device, dtype=torch.float32)
    Minv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
    Tm = Minv * af[..., None, :]
    W = Tm @ kf
    U = Tm @ vf
    P = torch.tril(qf @ kf.transpose(-1, -2))
    S = torch.zeros(B, H, dk, dv, dtype=torch.float32, device=k.device) if s0 is None \
        else s0.float().clone()
    outs = []
    for c in range(n):
        if resets is not None:
            S = S * (~resets[:, c].bool()).to(S.dtype).view(B, 1, 1, 1)
        Up = U[:, :, c] - W[:, :, c] @ S
        outs.append(qf[:, :, c] @ S + P[:, :, c] @ Up)
        S = S + kf[:, :, c].transpose(-1, -2) @ Up
    o = torch.stack(outs, dim=2)  # B,H,n,C,dv
    return o.permute(0, 2, 3, 1, 4).reshape(B, T, H, dv), S


def efla_reference_form(k, v, beta: float, s0=None, readout: str = "model"):
    """The reference's special case of the recurrence: q = k, one scalar beta, c_t from
    ||k_t||^2 (kernels/cuda/efla.cu:181-221) - the STATE recurrence is the reference's exactly.

    ``readout`` selects how the output is read from the state S (d_k x d_v, row = key index):

    * ``"model"`` (default): ``o_t = S_t^T k_t``, the contraction over the KEY index that this
      framework's model and kernels use (with a separate q in general);
    * ``"reference"``: ``o_t[row] = sum_col S_t[row][col] k_t[col]``, i.e. ``S_t k_t``, the
      contraction over the VALUE index that the reference's kernel and its CPU routine
      perform (kernels/cuda/efla.cu:222-231, ``eflaComputeOutput`` in
      src/kernels/efla_kernels.zig); it needs d_k = d_v.  The CUDA kernels of this framework
      do not implement this read-out: it exists here so that the difference is pinned by a
      test rather than by a docstring."""
    lam = k.float().pow(2).sum(-1)
    alpha = efla_coefficient(torch.full_like(lam, beta), lam)
    if readout == "model":
        return delta_rule_sequential(k, k, v, alpha, s0)
    if readout != "reference":
        raise ValueError(readout)
    B, T, H, d = k.shape
    assert v.shape[-1] == d, "the reference's read-out contracts keys with the value index"
    S = torch.zeros(B, H, d, d, dtype=torch.float32, device=k.device) if s0 is None \
        else s0.float().clone()
    kf, vf = k.float(), v.float()
    outs = []
    for t in range(T):
        kt, vt, a = kf[:, t], vf[:, t], alpha[:, t]
        u = torch.einsum("bhkv,bhk->bhv", S, kt)                      # S^T k
        S = S + a[..., None, None] * kt[..., :, None] * (vt - u)[..., None, :]
        outs.append(torch.einsum("bhrc,bhc->bhr", S, kt))              # S k (over columns)
    return torch.stack(outs, dim=1).to(k.dtype), S


# ---------------------------------------------------------------------- ShortConv / PRISM
def shortconv(x, weight):
    """Causal depthwise conv: y[t,d] = sum_w x[t-w,d] * W[d,w].  x: (B,T,D); weight: (D,Wn)."""
    B, T, D = x.shape
    Wn = weight.shape[1]
    xf = x.float().transpose(1, 2)  # B,D,T
    xp = F.pad(xf, (Wn - 1, 0))
    w = weight.float().flip(-1).unsqueeze(1)  # conv1d correlates: tap j hits x[t-(Wn-1-j)]
    y = F.conv1d(xp, w, groups=D)
    return y.transpose(1, 2).to(x.dtype)


# -------------------------------------------------------------------------- optimizers
def adamw_step(p, m, v, g, lr, b1, b2, eps, wd, step):
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    mh = m / (1 - b1**step)
    vh = v / (1 - b2**step)
    p.mul_(1 - lr * wd).sub_(lr * mh / (vh.sqrt() + eps))


def lion_step(p, m, g, lr, b1, b2, wd):
    u = b1 * m + (1 - b1) * g
    p.mul_(1 - lr * wd).sub_(lr * torch.sign(u))
    m.mul_(b2).add_(g, alpha=1 - b2)


def newton_schulz_cubic(y, iters):
    """Y <- 1/2 Y (3I - Y^T Y) on the Frobenius-normalised momentum
    (src/optim/optimizer.zig:253-319)."""
    y = y / (y.norm() + 1e-7)
    transposed = y.shape[0] < y.shape[1]
    if transposed:
        y = y.t()
    n = y.shape[1]
    eye = torch.eye(n, dtype=y.dtype, device=y.device)
    for _ in range(iters):
        y = 0.5 * y @ (3 * eye - y.t() @ y)
    return y.t() if transposed else y


def newton_schulz_quintic(g, iters=5):
    """The quintic iteration of the public Muon recipe (coefficients 3.4445, -4.7750, 2.0315)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g / (g.norm() + 1e-7)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    for _ in range(iters):
        A = x @ x.t()
        x = a * x + (b * A + c * A @ A) @ x
    return x.t() if transposed else x


def clip_scale(total_norm: float, max_norm: float) -> float:
    if max_norm <= 0 or not math.isfinite(total_norm):
        return 1.0 if math.isfinite(total_norm) else 0.0
    return min(1.0, max_norm / (total_norm + 1e-6))
