"""PRISM refinement branch and the causal depthwise ShortConv.

The reference specifies PRISM as an iterative residual refinement driven by a
short-convolution summary of the input (src/model/prism.zig:11-40):

    u = ShortConv(x);  r^1 = v - u;  for l = 1..L:  delta^l = GELU(p^l . r^l),
    r^(l+1) = r^l - delta^l,   with beta^l = W_beta^l u, k^l = W_k^l u, p^l = W_p^l u

but only ships a degenerate CPU loop (beta fixed at 0.5, p read from one weight row, no
state: prism.zig:279-320) and per-iteration weights of shape (hidden, head_dim)
(prism.zig:41-157).  This module implements the specified refinement in the head_dim-wide
proxy space those weight shapes imply:

    r_p = r W_k^l                      (residual seen through the proxy keys)
    delta = GELU((u W_p^l) * r_p)      (B,T,head_dim)
    c = (sigmoid(u W_beta^l) * delta) W_k^l^T      (back to hidden)
    r <- r - c ;   out <- out + forget_factor^(l-1) * c

with the gate and the update each one kernel (``ops/prism.py``, ``csrc/prism.cu``) and the
projections on the GEMM, and keeps the recurrent state the reference specifies,

    S_t = alpha S_{t-1} (I - b_t k_t^T) + sum_l (beta^l * delta^l) k^l^T,   b_t = beta^1 * k^1,

(k^l = u W_k^l, head_dim x head_dim per sequence) for generation: ``decode_step`` advances it
together with the ShortConv window, one token at a time.

ShortConv is y[t,d] = sum_w x[t-w,d] W[d,w] (prism.zig:448-476).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import conv as conv_ops
from ..ops import prism as P
from ..ops.matmul import linear


class ShortConv(nn.Module):
    def __init__(self, dim, window, device, dtype, gen):
        super().__init__()
        w = torch.empty(dim, window, device=device, dtype=torch.float32)
        w.normal_(0.0, (1.0 / window) ** 0.5, generator=gen)
        self.weight = nn.Parameter(w.to(dtype))

    def forward(self, x):
        return conv_ops.shortconv(x, self.weight)


class PrismLayer(nn.Module):
    def __init__(self, cfg, device, dtype, gen, std):
        super().__init__()
        p = cfg.prism
        self.L = p.num_iterations
        self.forget = p.forget_factor
        self.alpha = p.forget_factor  # the state's forget factor (prism.zig: alpha)
        D, hd = cfg.hidden_dim, cfg.head_dim
        self.hd = hd
        self.shortconv = ShortConv(D, p.shortconv_window, device, dtype, gen)

        def mk():
            t = torch.empty(hd, D, device=device, dtype=torch.float32)
            t.normal_(0.0, std, generator=gen)
            return nn.Parameter(t.to(dtype))
        self.w_beta = nn.ParameterList(mk() for _ in range(self.L))
        self.w_k = nn.ParameterList(mk() for _ in range(self.L))
        self.w_p = nn.ParameterList(mk() for _ in range(self.L))

    def forward(self, x_norm, a, state=None, return_state: bool = False):
        """x_norm: normed block input (B,T,D); a: EFLA branch output (B,T,D).
        Returns the refined branch output (to be added to the residual stream); with
        ``return_state`` also the recurrent state (B, hd, hd) fp32 after the T tokens, started
        from ``state`` (the reference's ``PrismState``, src/model/prism.zig:480-523):
        S_t = alpha S_{t-1} (I - b_t k_t^T) + sum_l bd_t^l k_t^l^T.  The ShortConv proxy stands
        in for the state's read-out (prism.zig:14-16), so the state never feeds the output and
        is only computed on request (generation, evaluation with carried state)."""
        u = self.shortconv(x_norm)
        out, bds, ks, bt1 = self._refine(u, a, return_state)
        if not return_state:
            return out
        B, T = x_norm.shape[:2]
        s = P.state(torch.stack(bds).view(self.L, B, T, self.hd),
                    torch.stack(ks).view(self.L, B, T, self.hd), bt1.view(B, T, self.hd), state,
                    self.alpha)
        return out, s

    def _refine(self, u, a, want_state_inputs: bool):
        r = a - u
        out = a
        scale = 1.0
        bds, ks, bt1 = [], [], None
        for l in range(self.L):
            rp = linear(r, self.w_k[l])
            p = linear(u, self.w_p[l])
            bt = linear(u, self.w_beta[l])
            bd = P.gate(rp, p, bt)                       # sigmoid(bt) * GELU(p * rp)
            c = _matmul_nn(bd, self.w_k[l])              # (B,T,hd) x (hd,D): back to hidden
            r, out = P.update(c, r, out, scale)          # r - c, out + scale * c
            scale *= self.forget
            if want_state_inputs:
                bds.append(bd.detach())
                ks.append(linear(u, self.w_k[l]).detach())
                if l == 0:
                    bt1 = bt.detach()
        return out, bds, ks, bt1

    # ------------------------------------------------------------------ recurrent decode
    def new_cache(self, batch: int, device=None, dtype=None):
        """Per-sequence decode state: the last ``window - 1`` block inputs (for the causal
        ShortConv) and the recurrent state S."""
        w = self.shortconv.weight
        device = device or w.device
        return {"conv": torch.zeros(batch, w.shape[1] - 1, w.shape[0], device=device,
                                    dtype=dtype or w.dtype),
                "state": torch.zeros(batch, self.hd, self.hd, dtype=torch.float32, device=device)}

    @torch.no_grad()
    def decode_step(self, x_norm, a, cache):
        """One token: x_norm, a: (B, D).  Updates ``cache`` in place; returns the refined
        branch output (B, D), equal to the corresponding row of ``forward`` on the prefix."""
        w = self.shortconv.weight                         # (D, window): y[t] = sum_j x[t-j] w[:, j]
        hist = torch.cat([cache["conv"], x_norm[:, None, :].to(cache["conv"].dtype)], dim=1)
        win = hist.shape[1]
        taps = w.float().t().flip(0)[-win:]               # oldest input first
        u = (hist.float() * taps[None]).sum(1).to(x_norm.dtype)
        cache["conv"] = hist[:, 1:] if win == w.shape[1] else hist
        out, bds, ks, bt1 = self._refine(u, a, True)
        B = x_norm.shape[0]
        cache["state"] = P.state(torch.stack(bds).view(self.L, B, 1, self.hd),
                                 torch.stack(ks).view(self.L, B, 1, self.hd),
                                 bt1.view(B, 1, self.hd), cache["state"], self.alpha)
        return out

    def reference_tensors(self):
        out = {"shortconv.weight": self.shortconv.weight.detach()}
        for j in range(self.L):
            out[f"w_beta.{j}"] = self.w_beta[j].detach().t().contiguous()
            out[f"w_k.{j}"] = self.w_k[j].detach().t().contiguous()
            out[f"w_p.{j}"] = self.w_p[j].detach().t().contiguous()
        return out

    @torch.no_grad()
    def load_reference_tensors(self, t):
        self.shortconv.weight.copy_(t["shortconv.weight"].to(self.shortconv.weight))
        for j in range(self.L):
            self.w_beta[j].copy_(t[f"w_beta.{j}"].t().to(self.w_beta[j]))
            self.w_k[j].copy_(t[f"w_k.{j}"].t().to(self.w_k[j]))
            self.w_p[j].copy_(t[f"w_p.{j}"].t().to(self.w_p[j]))


class _MatmulNN(torch.autograd.Function):
    """y = x @ w with w of shape (K, N) (the transposed use of a projection weight)."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops.matmul import gemm
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, w)
        ctx.wref = w
        ctx.shape = x.shape
        return gemm(x2, w, b_mn=True).view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        from ..ops.matmul import gemm
        x2, _ = ctx.saved_tensors
        w = ctx.wref
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = gemm(dy2, w).view(ctx.shape)                       # dy (M,N) . w^T (N,K)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            gemm(x2, dy2, a_mn=True, b_mn=True, out=mg, accumulate=True)  # x^T dy -> (K,N)
            w.grad_touched = True
            return dx, None
        return dx, gemm(x2, dy2, a_mn=True, b_mn=True, out_dtype=w.dtype)


def _matmul_nn(x, w):
    return _MatmulNN.apply(x, w)
