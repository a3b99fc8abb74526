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

ShortConv is y[t,d] = sum_w x[t-w,d] W[d,w] (prism.zig:448-476).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import conv as conv_ops
from ..ops import nn as K
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

    def forward(self, x_norm, a):
        """x_norm: normed block input (B,T,D); a: EFLA branch output (B,T,D).
        Returns the refined branch output (to be added to the residual stream)."""
        u = self.shortconv(x_norm)
        r = a - u
        out = a
        scale = 1.0
        for l in range(self.L):
            rp = linear(r, self.w_k[l])
            p = linear(u, self.w_p[l])
            b = torch.sigmoid(linear(u, self.w_beta[l]).float())
            delta = K.activation((p.float() * rp.float()).to(a.dtype), "gelu")
            bd = (b * delta.float()).to(a.dtype)
            c = _matmul_nn(bd, self.w_k[l])  # (B,T,hd) x (hd,D)
            r = r - c
            out = out + scale * c
            scale *= self.forget
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
