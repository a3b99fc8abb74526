"""The EFLA language model under tensor parallelism (with sequence-sharded activations) and
context parallelism.

Tensor parallel (``tp``): heads and MLP columns are split over the group; between the
row-parallel and column-parallel GEMMs the residual stream lives as a row shard
(tokens / tp rows per rank), norms run on the shard, and the two collectives per sub-layer are
fused into the GEMM kernels (``parallel/tp.py``: all-gather -> QKV / up GEMM, out / down GEMM
-> reduce-scatter + residual).  EFLA itself needs no communication: its state is per head.

Context parallel (``cp``): each rank holds a contiguous span of every sequence; all layers
are local except the EFLA recurrence, which exchanges affine state maps (``parallel/cp.py``).

Weights are cut out of the same full-size random tensors ``EflaLM`` draws (same seed), so a
parallel model and the single-GPU model are the same function.  Parameters every rank of a
group holds in full (norms, embeddings, LM head) carry ``replicated = True``; their gradients
must be summed over that group before the optimizer step (``sync_replicated_grads``).

The reference describes these layouts (src/tensor/sharding.zig:183-287) and runs none.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import efla as efla_ops
from ..ops import nn as K
from ..ops.matmul import linear
from ..parallel.cp import cp_delta_rule
from ..parallel.tp import column_parallel_linear, row_parallel_linear
from ..utils.config import ModelConfig
from .model import Norm


def _full(shape, std, device, gen):
    t = torch.empty(shape, device=device, dtype=torch.float32)
    t.normal_(0.0, std, generator=gen)
    return t


def _shard_rows(t, parts, rank, world):
    """t: (parts*rows, K) laid out as `parts` equal blocks; returns this rank's slice of each."""
    blocks = t.chunk(parts, dim=0)
    return torch.cat([b.chunk(world, dim=0)[rank] for b in blocks], dim=0)


class ParallelBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, device, gen, std, tp_rank, tp_world):
        super().__init__()
        if cfg.prism.enabled:
            raise ValueError("the PRISM branch is not available under tensor/context parallelism")
        if cfg.activation != "swiglu" and cfg.activation not in K.ACT_MODES:
            raise ValueError(cfg.activation)
        e = cfg.efla
        dt = torch.bfloat16
        D, H, d, F = cfg.hidden_dim, cfg.num_heads, cfg.head_dim, cfg.intermediate_dim
        assert H % tp_world == 0 and F % tp_world == 0
        self.H_loc, self.d, self.D, self.F_loc = H // tp_world, d, D, F // tp_world
        self.P = 3 if e.use_query else 2
        self.normalize, self.per_token_beta = e.normalize_qk, e.per_token_beta
        self.act = cfg.activation
        self.ln1 = Norm(D, cfg.norm_type, device, dt)
        self.ln2 = Norm(D, cfg.norm_type, device, dt)
        for n in (self.ln1, self.ln2):
            for p in n.parameters():
                p.replicated = True
        # draw the full tensors in EflaLM's order, keep this rank's slice
        w_qkv = _full((self.P * H * d, D), std, device, gen)
        w_o = _full((D, H * d), std, device, gen)
        w_loc = _shard_rows(w_qkv, self.P, tp_rank, tp_world)
        self.w_o = nn.Parameter(w_o.chunk(tp_world, dim=1)[tp_rank].contiguous().to(dt))
        if self.per_token_beta:
            w_beta = _full((H, D), std, device, gen).chunk(tp_world, dim=0)[tp_rank]
            pad = (-(w_loc.shape[0] + self.H_loc)) % 64
            w_loc = torch.cat([w_loc, w_beta, torch.zeros(pad, D, device=device)])
            self.qkv_pad_rows = pad
            self.beta_param = None
        else:
            self.qkv_pad_rows = 0
            self.beta_param = nn.Parameter(torch.full((1,), float(e.initial_beta), device=device),
                                           requires_grad=e.learned_beta)
            self.beta_param.replicated = True
        self.w_qkv = nn.Parameter(w_loc.to(dt).contiguous())
        parts = 2 if self.act == "swiglu" else 1
        w_up = _full((parts * F, D), std, device, gen)
        w_down = _full((D, F), std, device, gen)
        self.w_up = nn.Parameter(_shard_rows(w_up, parts, tp_rank, tp_world).to(dt))
        self.w_down = nn.Parameter(w_down.chunk(tp_world, dim=1)[tp_rank].contiguous().to(dt))

    def _attention(self, proj, B, T, cp):
        hd = self.H_loc * self.d
        proj = proj.view(B, T, -1)
        if cp is None:
            if self.per_token_beta:
                return efla_ops.efla_proj(proj, self.P, self.H_loc, self.d, self.normalize)[0]
            return efla_ops.efla_qkv(proj.view(B, T, self.P, self.H_loc, self.d), self.beta_param,
                                     self.normalize)[0]
        qkv = proj[..., :self.P * hd].reshape(B, T, self.P, self.H_loc, self.d)
        beta = torch.sigmoid(proj[..., self.P * hd:self.P * hd + self.H_loc].float()) \
            if self.per_token_beta else self.beta_param
        q = qkv[:, :, 0]
        k = qkv[:, :, 1] if self.P == 3 else qkv[:, :, 0]
        v = qkv[:, :, self.P - 1]
        if self.normalize:
            q, k = efla_ops.l2norm(q), efla_ops.l2norm(k)
            alpha = -torch.expm1(-beta.float().expand(B, T, self.H_loc))
        else:
            alpha = efla_ops.ref.efla_coefficient(beta.float().expand(B, T, self.H_loc),
                                                  k.float().pow(2).sum(-1))
        return cp_delta_rule(q, k, v, alpha, cp)

    def forward(self, h, B, T, tp=None, cp=None, impl="fused"):
        """h: (rows, D) - all B*T local tokens without tp, this rank's row shard with tp."""
        n1, h = self.ln1(h, skip=True)
        proj = column_parallel_linear(n1, self.w_qkv, tp, impl) if tp is not None \
            else linear(n1, self.w_qkv)
        o = self._attention(proj, B, T, cp).reshape(B * T, self.H_loc * self.d)
        if tp is not None:
            h = row_parallel_linear(o, self.w_o, tp, residual=h, impl=impl)
            n2, h = self.ln2(h, skip=True)
            u = column_parallel_linear(n2, self.w_up, tp, impl)
        else:
            h = linear(o, self.w_o, h)
            n2, h = self.ln2(h, skip=True)
            u = linear(n2, self.w_up)
        a = K.swiglu(u) if self.act == "swiglu" else K.activation(u, self.act)
        if tp is not None:
            return row_parallel_linear(a, self.w_down, tp, residual=h, impl=impl)
        return linear(a, self.w_down, h)


class ParallelEflaLM(nn.Module):
    """``tp``: a ``TPContext`` (or None); ``cp``: a ``CPContext`` (or None).  ``forward`` takes
    the tokens of this rank's data-parallel replica: the full (B, T) batch under tp (every tp
    rank passes the same tensors), this rank's (B, T/cp) span under cp."""

    def __init__(self, cfg: ModelConfig, device, tp=None, cp=None, seed: int = 0,
                 init_std: float = 0.02, impl: str = "fused"):
        super().__init__()
        self.cfg, self.tp, self.cp, self.impl = cfg, tp, cp, impl
        device = torch.device(device)
        tp_rank, tp_world = (tp.rank, tp.world) if tp is not None else (0, 1)
        self.tp_rank, self.tp_world = tp_rank, tp_world
        gen = torch.Generator(device=device).manual_seed(seed)
        dt = torch.bfloat16
        self.embed_tokens = nn.Parameter(_full((cfg.vocab_size, cfg.hidden_dim), init_std, device,
                                               gen).to(dt))
        self.embed_tokens.replicated = True
        self.blocks = nn.ModuleList(ParallelBlock(cfg, device, gen, init_std, tp_rank, tp_world)
                                    for _ in range(cfg.num_layers))
        self.final_norm = Norm(cfg.hidden_dim, cfg.norm_type, device, dt)
        for p in self.final_norm.parameters():
            p.replicated = True
        self.lm_head = None
        if not cfg.tie_embeddings:
            self.lm_head = nn.Parameter(_full((cfg.vocab_size, cfg.hidden_dim), init_std, device,
                                              gen).to(dt))
            self.lm_head.replicated = True

    def forward(self, tokens, targets, label_smoothing: float = 0.0):
        B, T = tokens.shape
        tok, tgt = tokens.reshape(-1), targets.reshape(-1)
        if self.tp is not None:  # sequence-parallel: this rank embeds and scores its row shard
            rows = tok.numel() // self.tp_world
            sl = slice(self.tp_rank * rows, (self.tp_rank + 1) * rows)
            tok, tgt = tok[sl], tgt[sl]
        h = K.embedding(tok, self.embed_tokens)
        for blk in self.blocks:
            h = blk(h, B, T, self.tp, self.cp, self.impl)
        hn = self.final_norm(h)
        w = self.embed_tokens if self.lm_head is None else self.lm_head
        return K.linear_cross_entropy(hn, w, tgt, label_smoothing)

    # ------------------------------------------------------------ checkpoint name mapping
    def state_dict_shards(self):
        """This rank's tensors under the reference's names and (in, out) orientation
        (src/model/model.zig:494-521), as ``name -> (tensor, shard_dim)``: ``shard_dim`` is the
        dimension of the FULL tensor this rank holds a ``1 / tp`` slice of (its tp rank-th
        slice), or None for a tensor every rank holds whole."""
        out = {}
        out["embed_tokens.weight"] = (self.embed_tokens.detach(), None)
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}."
            hd = b.H_loc * b.d
            out[p + "ln1.weight"] = (b.ln1.weight.detach(), None)
            if b.ln1.bias is not None:
                out[p + "ln1.bias"] = (b.ln1.bias.detach(), None)
            names = ["w_q", "w_k", "w_v"] if b.P == 3 else ["w_k", "w_v"]
            for j, nme in enumerate(names):
                out[p + "efla." + nme] = (b.w_qkv.detach()[j * hd:(j + 1) * hd].t().contiguous(), 1)
            out[p + "efla.w_o"] = (b.w_o.detach().t().contiguous(), 0)
            if b.per_token_beta:
                nb = len(names) * hd
                out[p + "efla.w_beta"] = (b.w_qkv.detach()[nb:nb + b.H_loc].t().contiguous(), 1)
            else:
                out[p + "efla.beta_param"] = (b.beta_param.detach(), None)
            out[p + "ln2.weight"] = (b.ln2.weight.detach(), None)
            if b.ln2.bias is not None:
                out[p + "ln2.bias"] = (b.ln2.bias.detach(), None)
            if b.act == "swiglu":
                g, u = b.w_up.detach().split(b.F_loc, dim=0)
                out[p + "mlp_gate.weight"] = (g.t().contiguous(), 1)
                out[p + "mlp_up.weight"] = (u.t().contiguous(), 1)
            else:
                out[p + "mlp_up.weight"] = (b.w_up.detach().t().contiguous(), 1)
            out[p + "mlp_down.weight"] = (b.w_down.detach().t().contiguous(), 0)
        out["final_norm.weight"] = (self.final_norm.weight.detach(), None)
        if self.final_norm.bias is not None:
            out["final_norm.bias"] = (self.final_norm.bias.detach(), None)
        if self.lm_head is not None:
            out["lm_head.weight"] = (self.lm_head.detach().t().contiguous(), None)
        return out

    @torch.no_grad()
    def load_reference_state(self, tensors: dict) -> None:
        """Loads FULL tensors (reference names and orientation, e.g. a checkpoint written at
        any tensor-parallel size) and keeps this rank's slices."""
        r, w = self.tp_rank, self.tp_world

        def put(dst, src):
            dst.copy_(src.to(dst.device, dst.dtype))

        def cut(t, dim):
            return t.chunk(w, dim=dim)[r]
        put(self.embed_tokens, tensors["embed_tokens.weight"])
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}."
            hd = b.H_loc * b.d
            put(b.ln1.weight, tensors[p + "ln1.weight"])
            if b.ln1.bias is not None:
                put(b.ln1.bias, tensors[p + "ln1.bias"])
            names = ["w_q", "w_k", "w_v"] if b.P == 3 else ["w_k", "w_v"]
            for j, nme in enumerate(names):
                put(b.w_qkv[j * hd:(j + 1) * hd], cut(tensors[p + "efla." + nme], 1).t())
            put(b.w_o, cut(tensors[p + "efla.w_o"], 0).t())
            if b.per_token_beta:
                nb = len(names) * hd
                put(b.w_qkv[nb:nb + b.H_loc], cut(tensors[p + "efla.w_beta"], 1).t())
            else:
                put(b.beta_param, tensors[p + "efla.beta_param"].reshape(1))
            put(b.ln2.weight, tensors[p + "ln2.weight"])
            if b.ln2.bias is not None:
                put(b.ln2.bias, tensors[p + "ln2.bias"])
            if b.act == "swiglu":
                put(b.w_up[:b.F_loc], cut(tensors[p + "mlp_gate.weight"], 1).t())
                put(b.w_up[b.F_loc:], cut(tensors[p + "mlp_up.weight"], 1).t())
            else:
                put(b.w_up, cut(tensors[p + "mlp_up.weight"], 1).t())
            put(b.w_down, cut(tensors[p + "mlp_down.weight"], 0).t())
        put(self.final_norm.weight, tensors["final_norm.weight"])
        if self.final_norm.bias is not None:
            put(self.final_norm.bias, tensors["final_norm.bias"])
        if self.lm_head is not None:
            put(self.lm_head, tensors["lm_head.weight"].t())

    def count_parameters(self) -> int:
        """Parameters of the whole model (sharded tensors counted at full size)."""
        n = 0
        for p in self.parameters():
            n += p.numel() if getattr(p, "replicated", False) else p.numel() * self.tp_world
        return n

    def grad_scale_divisor(self) -> int:
        """Each rank of a tp / cp group back-propagates the mean loss of ITS tokens; the
        gradient of the group's mean loss is the sum of those divided by the group size."""
        d = self.tp_world
        if self.cp is not None:
            d *= self.cp.world
        return d

    def flops_per_token(self, seq_len=None) -> float:
        c = self.cfg
        mat = sum(p.numel() for n, p in self.named_parameters() if p.dim() == 2
                  and "embed_tokens" not in n and not getattr(p, "replicated", False))
        mat -= sum(b.qkv_pad_rows * c.hidden_dim for b in self.blocks)  # zero padding rows
        mat *= self.tp_world
        mat += (self.embed_tokens if self.lm_head is None else self.lm_head).numel()
        efla = c.num_layers * c.num_heads * (4 * c.head_dim * c.head_dim + 8 * 64 * c.head_dim)
        return 6.0 * mat + 3.0 * efla


def sync_replicated_grads(model: nn.Module, group) -> None:
    """Sum the ``main_grad`` (or ``grad``) of replicated parameters over ``group``."""
    if group is None or dist.get_world_size(group) == 1:
        return
    for p in model.parameters():
        if getattr(p, "replicated", False):
            g = getattr(p, "main_grad", None)
            if g is None:
                g = p.grad
            if g is not None:
                dist.all_reduce(g, group=group)
