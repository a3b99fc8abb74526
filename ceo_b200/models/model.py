"""EFLA decoder language model.

Block (pre-norm, residual), following the reference's TransformerBlock
(src/model/model.zig:152-204) with the generalisations its configs name:

    h += W_o . EFLA(qkv(norm1 h))            [+ PRISM refinement when enabled]
    h += W_down . act(W_up norm2 h)          (SwiGLU when activation = swiglu)

The residual adds ride in the epilogue of the out-proj / down-proj GEMMs; q/k/v (and the
gate/up pair) come from one fused projection each.  Parameter names on disk follow the
reference (model.zig:494-521: ``embed_tokens.weight``, ``blocks.{i}.ln1.weight``,
``blocks.{i}.efla.{w_k,w_v,w_o,beta_param}``, ``blocks.{i}.mlp_up.weight`` ...) with the
additions ``efla.w_q``, ``efla.w_beta`` and ``mlp_gate.weight``; ``state_dict_reference()``
/ ``load_reference_state()`` translate between the fused (out, in) tensors kept here and
the per-matrix (in, out) tensors of the checkpoint format (src/nn/layers.zig:509,529).
"""
from __future__ import annotations

import functools
import math
from collections import OrderedDict

import torch
import torch.nn as nn

from ..ops import efla as efla_ops
from ..ops import nn as K
from ..ops.fp8 import Fp8Recipe, fp8_linear
from ..ops import matmul as matmul_ops
from ..ops.matmul import linear
from ..utils.config import ModelConfig
from .prism import PrismLayer


def _param(shape, std, device, dtype, gen):
    t = torch.empty(shape, device=device, dtype=torch.float32)
    if std == 0.0:
        t.zero_()
    else:
        t.normal_(0.0, std, generator=gen)
    return nn.Parameter(t.to(dtype))


def _lin(mod, name, x, w, residual=None):
    """The module's Linear ``name``: on e4m3 operands when FP8 training is enabled for it
    (``EflaLM.enable_fp8``), in bf16 otherwise."""
    st = mod.fp8
    if st is None:
        return linear(x, w, residual)
    return fp8_linear(x, w, st[name], residual)


class _StateList(list):
    """The per-block EFLA states; a list that can also carry the PRISM decode caches."""
    prism = None


class Norm(nn.Module):
    def __init__(self, dim, kind, device, dtype):
        super().__init__()
        self.kind = kind
        self.eps = 1e-6 if kind == "rmsnorm" else 1e-5
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype)) \
            if kind == "layernorm" else None

    def forward(self, x, skip: bool = False):
        """``skip=True`` returns ``(y, x_skip)``: use ``x_skip`` where the residual stream goes
        on (RMSNorm folds the gradient add into its backward kernel)."""
        if self.kind == "rmsnorm":
            y, xs = K.rmsnorm(x, self.weight, self.eps, skip=skip)
            return (y, xs) if skip else y
        y = K.layernorm(x, self.weight, self.bias, self.eps)
        return (y, x) if skip else y


class EflaLayer(nn.Module):
    """Projections + EFLA attention (reference: src/model/efla.zig:110-249)."""

    def __init__(self, cfg: ModelConfig, device, dtype, gen, std):
        super().__init__()
        e = cfg.efla
        self.H, self.d, self.D = cfg.num_heads, cfg.head_dim, cfg.hidden_dim
        self.P = 3 if e.use_query else 2
        self.normalize = e.normalize_qk
        self.per_token_beta = e.per_token_beta
        hd = self.H * self.d
        self.hd = hd
        w_qkv = _param((self.P * hd, self.D), std, device, dtype, gen).data
        self.w_o = _param((self.D, hd), std, device, dtype, gen)
        if self.per_token_beta:
            # the beta logits ride in the same projection: rows [q | k | v | beta (H) | zero pad];
            # padded to a multiple of 64 rows so the weight-gradient GEMM can fetch the operand
            # tile with one TMA request per stage
            w_beta = _param((self.H, self.D), std, device, dtype, gen).data
            pad = (-(self.P * hd + self.H)) % 64
            w_qkv = torch.cat([w_qkv, w_beta, torch.zeros(pad, self.D, device=device, dtype=dtype)])
            self.beta_param = None
        else:
            self.beta_param = nn.Parameter(torch.full((1,), float(e.initial_beta), device=device,
                                                      dtype=torch.float32),
                                           requires_grad=e.learned_beta)
        self.qkv_pad_rows = w_qkv.shape[0] - self.P * hd - (self.H if self.per_token_beta else 0)
        self.w_qkv = nn.Parameter(w_qkv)
        self.fp8 = None

    def forward(self, x_norm, residual, state=None, resets=None):
        B, T, _ = x_norm.shape
        if (-T) % efla_ops.CHUNK and x_norm.is_cuda:
            raise ValueError(f"sequence length {T} must be a multiple of {efla_ops.CHUNK} on GPU")
        proj = _lin(self, "qkv", x_norm, self.w_qkv)
        if self.per_token_beta:
            o, s_final = efla_ops.efla_proj(proj, self.P, self.H, self.d, self.normalize, state,
                                            resets)
        else:
            o, s_final = efla_ops.efla_qkv(proj.view(B, T, self.P, self.H, self.d),
                                           self.beta_param, self.normalize, state, resets)
        return o.reshape(B, T, self.H * self.d), s_final

    def decode_step(self, x_norm, state):
        """One token (B, D) with carried state (B,H,d,d) fp32; returns the (B, H*d) output."""
        B = x_norm.shape[0]
        proj = linear(x_norm, self.w_qkv)
        qkv = proj[:, :self.P * self.hd].reshape(B, self.P, self.H, self.d)
        q = qkv[:, 0]
        k = qkv[:, 1] if self.P == 3 else qkv[:, 0]
        v = qkv[:, self.P - 1]
        if self.per_token_beta:
            beta = torch.sigmoid(proj[:, self.P * self.hd:self.P * self.hd + self.H].float())
        else:
            beta = self.beta_param.expand(B, self.H)
        if self.normalize:
            q, k = efla_ops.l2norm(q), efla_ops.l2norm(k)
            alpha = -torch.expm1(-beta)
        else:
            alpha = efla_ops.ref.efla_coefficient(beta, k.float().pow(2).sum(-1))
        o = efla_ops.delta_rule_decode_step(q, k, v, alpha, state)
        return o.reshape(B, self.H * self.d)


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, device, dtype, gen, std):
        super().__init__()
        self.act = cfg.activation
        D, F = cfg.hidden_dim, cfg.intermediate_dim
        self.F = F
        n_up = 2 * F if self.act == "swiglu" else F
        self.w_up = _param((n_up, D), std, device, dtype, gen)
        if self.act == "swiglu":
            # drawn as [gate | up] row blocks, kept INTERLEAVED (row 2j = gate_j, row 2j+1 =
            # up_j): an output tile of the gate/up GEMM then holds matching (gate, up) pairs
            # and its epilogue can apply SiLU(gate) * up
            w = self.w_up.data
            self.w_up.data = w.view(2, F, D).transpose(0, 1).reshape(n_up, D).contiguous()
        self.w_down = _param((D, F), std, device, dtype, gen)
        self.fp8 = None

    def gate_up_weights(self):
        """(W_gate, W_up), each (F, D) (strided views of the interleaved parameter)."""
        return self.w_up[0::2], self.w_up[1::2]

    def forward(self, x_norm, residual):
        if self.act == "swiglu":
            if x_norm.is_cuda and self.fp8 is None and matmul_ops.FUSED_SWIGLU and self.F % 32 == 0:
                return matmul_ops.swiglu_mlp(x_norm, self.w_up, self.w_down, residual)
            a = K.swiglu(_lin(self, "up", x_norm, self.w_up), interleaved=True)
        else:
            a = K.activation(_lin(self, "up", x_norm, self.w_up), self.act)
        return _lin(self, "down", a, self.w_down, residual)


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig, device, dtype, gen, std):
        super().__init__()
        self.ln1 = Norm(cfg.hidden_dim, cfg.norm_type, device, dtype)
        self.efla = EflaLayer(cfg, device, dtype, gen, std)
        self.prism = PrismLayer(cfg, device, dtype, gen, std) if cfg.prism.enabled else None
        self.ln2 = Norm(cfg.hidden_dim, cfg.norm_type, device, dtype)
        self.mlp = MLP(cfg, device, dtype, gen, std)
        self.dropout = float(cfg.dropout)  # on both branch outputs, training mode only

    def forward(self, h, state=None, resets=None):
        drop = self.dropout if self.training else 0.0
        n1, h = self.ln1(h, skip=True)
        o, s_final = self.efla(n1, h, state, resets)
        if self.prism is not None:
            a = _lin(self.efla, "o", o, self.efla.w_o)
            h = h + K.dropout(self.prism(n1, a), drop)
        elif drop > 0.0:
            h = h + K.dropout(_lin(self.efla, "o", o, self.efla.w_o), drop)
        else:
            h = _lin(self.efla, "o", o, self.efla.w_o, h)  # residual add in the GEMM epilogue
        n2, h = self.ln2(h, skip=True)
        if drop > 0.0:
            h = h + K.dropout(self.mlp(n2, None), drop)
        else:
            h = self.mlp(n2, h)
        return h, s_final

    def decode_step(self, h, state, prism_cache=None):
        n1 = self.ln1(h)
        o = self.efla.decode_step(n1, state)
        if self.prism is not None:
            if prism_cache is None:
                raise ValueError("a block with PRISM needs its decode cache "
                                 "(EflaLM.new_prism_caches)")
            h = h + self.prism.decode_step(n1, linear(o, self.efla.w_o), prism_cache)
        else:
            h = linear(o, self.efla.w_o, h)
        return self.mlp(self.ln2(h), h)


class EflaLM(nn.Module):
    """embed -> blocks -> final norm -> LM head (reference: src/model/model.zig:271-441)."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype=None, seed: int = 0,
                 init_std: float = 0.02):
        super().__init__()
        self.cfg = cfg
        if dtype is None:
            dtype = {"fp32": torch.float32, "fp16": torch.float16}.get(cfg.dtype, torch.bfloat16)
        device = torch.device(device)
        if device.type == "cuda" and dtype != torch.bfloat16:
            raise ValueError("the CUDA kernels are bf16; use dtype bf16 on GPU")
        gen = torch.Generator(device=device).manual_seed(seed)
        self.embed_tokens = _param((cfg.vocab_size, cfg.hidden_dim), init_std, device, dtype, gen)
        self.blocks = nn.ModuleList(Block(cfg, device, dtype, gen, init_std)
                                    for _ in range(cfg.num_layers))
        self.final_norm = Norm(cfg.hidden_dim, cfg.norm_type, device, dtype)
        self.lm_head = None if cfg.tie_embeddings else \
            _param((cfg.vocab_size, cfg.hidden_dim), init_std, device, dtype, gen)

        self.fp8_recipe = None
        # optional callable (block index, grad) -> grad, registered on every block's input
        self.block_input_hook = None

    def enable_fp8(self, history: int = 16, margin: int = 0, dgrad: bool = False,
                   wgrad: bool = False) -> Fp8Recipe:
        """Switches the four projections of every block (qkv, out, up / gate-up, down) to the
        FP8 forward product with per-tensor delayed scaling; the embedding, the norms, EFLA
        itself and the LM head stay in bf16; ``dgrad`` / ``wgrad`` also move their data /
        weight gradients to 8-bit operands (e5m2 dy).  The caller invokes ``recipe.step()`` after every optimizer
        step."""
        rec = Fp8Recipe(history, margin, dgrad, wgrad)
        dev = self.embed_tokens.device
        for blk in self.blocks:
            blk.efla.fp8 = {"qkv": rec.new_state(dev), "o": rec.new_state(dev)}
            blk.mlp.fp8 = {"up": rec.new_state(dev), "down": rec.new_state(dev)}
        self.fp8_recipe = rec
        return rec

    # ------------------------------------------------------------------ forward paths
    def head_weight(self):
        return self.embed_tokens if self.lm_head is None else self.lm_head

    def hidden(self, tokens, states=None, resets=None):
        h = K.embedding(tokens, self.embed_tokens)
        finals = []
        for i, blk in enumerate(self.blocks):
            if self.block_input_hook is not None and h.requires_grad:
                # fires in the backward pass once block i has produced all its gradients
                h.register_hook(functools.partial(self.block_input_hook, i))
            h, s = blk(h, None if states is None else states[i], resets)
            finals.append(s)
        return self.final_norm(h), finals

    def forward(self, tokens, targets=None, label_smoothing: float = 0.0, states=None,
                return_states: bool = False, resets=None):
        """With ``targets``: mean next-token cross-entropy (the LM head and the loss are fused,
        logits are never materialised; targets equal to -100 are left out).  Without: logits
        (B,T,V) in fp32.  ``resets`` (B, T/64): chunks that start a new document of a packed
        batch (``data.dataset.pack_sequences(..., align=64)``); the EFLA state is zeroed there."""
        hn, finals = self.hidden(tokens, states, resets)
        if targets is not None:
            out = K.linear_cross_entropy(hn, self.head_weight(), targets, label_smoothing)
        else:
            from ..ops.matmul import gemm
            w = self.head_weight()
            if hn.is_cuda:
                out = gemm(hn.reshape(-1, hn.shape[-1]), w, out_dtype=torch.float32)
            else:
                out = hn.reshape(-1, hn.shape[-1]).float() @ w.float().t()
            out = out.view(*tokens.shape, -1)
        return (out, finals) if return_states else out

    def new_states(self, batch, device=None):
        device = device or self.embed_tokens.device
        c = self.cfg
        return _StateList(torch.zeros(batch, c.num_heads, c.head_dim, c.head_dim,
                                      dtype=torch.float32, device=device) for _ in self.blocks)

    def new_prism_caches(self, batch, device=None):
        """Per-block PRISM decode caches (ShortConv window + recurrent state); None for blocks
        without the PRISM branch."""
        device = device or self.embed_tokens.device
        return [blk.prism.new_cache(batch, device) if blk.prism is not None else None
                for blk in self.blocks]

    @torch.no_grad()
    def decode_step(self, token, states, prism_caches=None):
        """token: (B,) ids; states: list of (B,H,d,d) fp32 updated in place -> logits (B,V).
        With the PRISM branch enabled the caches live next to the states: they are attached to
        the ``states`` list on first use (``states.prism``) unless passed explicitly."""
        if prism_caches is None and any(b.prism is not None for b in self.blocks):
            prism_caches = getattr(states, "prism", None)
            if prism_caches is None:
                prism_caches = self.new_prism_caches(token.shape[0], token.device)
                try:
                    states.prism = prism_caches
                except AttributeError:  # a plain list cannot carry the caches
                    raise ValueError("pass prism_caches=model.new_prism_caches(batch) to "
                                     "decode_step, or create the states with new_states()")
        if prism_caches is None:
            prism_caches = [None] * len(self.blocks)
        h = K.embedding(token, self.embed_tokens)
        for blk, st, pc in zip(self.blocks, states, prism_caches):
            h = blk.decode_step(h, st, pc)
        hn = self.final_norm(h)
        w = self.head_weight()
        if hn.is_cuda:
            from ..ops.matmul import gemm
            return gemm(hn, w, out_dtype=torch.float32)   # (B, V) logits on the tcgen05 GEMM
        return hn.float() @ w.float().t()

    # ------------------------------------------------------------ checkpoint name mapping
    def count_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def state_dict_reference(self) -> "OrderedDict[str, torch.Tensor]":
        """Tensors under the reference's names and (in, out) orientation."""
        out = OrderedDict()
        out["embed_tokens.weight"] = self.embed_tokens.detach()
        for i, b in enumerate(self.blocks):
            block_reference_tensors(b, f"blocks.{i}.", self.cfg, out)
        out["final_norm.weight"] = self.final_norm.weight.detach()
        if self.final_norm.bias is not None:
            out["final_norm.bias"] = self.final_norm.bias.detach()
        if self.lm_head is not None:
            out["lm_head.weight"] = self.lm_head.detach().t().contiguous()
        return out

    @torch.no_grad()
    def load_reference_state(self, tensors: dict) -> None:
        """Inverse of ``state_dict_reference`` (raises KeyError on a missing tensor)."""
        _put(self.embed_tokens, tensors["embed_tokens.weight"])
        for i, b in enumerate(self.blocks):
            load_block_reference(b, f"blocks.{i}.", self.cfg, tensors)
        _put(self.final_norm.weight, tensors["final_norm.weight"])
        if self.final_norm.bias is not None:
            _put(self.final_norm.bias, tensors["final_norm.bias"])
        if self.lm_head is not None:
            _put(self.lm_head, tensors["lm_head.weight"].t())

    def flops_per_token(self, seq_len: int | None = None) -> float:
        """Model FLOPs per token for one forward+backward (6 x matmul parameters + EFLA)."""
        c = self.cfg
        mat = sum(p.numel() for n, p in self.named_parameters() if p.dim() == 2
                  and "embed_tokens" not in n)
        mat -= sum(b.efla.qkv_pad_rows * c.hidden_dim for b in self.blocks)  # zero padding rows
        if self.lm_head is None:
            mat += self.embed_tokens.numel()
        efla = c.num_layers * c.num_heads * (4 * c.head_dim * c.head_dim + 8 * 64 * c.head_dim)
        return 6.0 * mat + 3.0 * efla


def model_flops_per_token(c: ModelConfig) -> float:
    """Model FLOPs per token of one forward + backward, from the configuration alone
    (6 x the multiply-accumulates of the projections, MLP and LM head, plus EFLA)."""
    e = c.efla
    hd = c.num_heads * c.head_dim
    P = 3 if e.use_query else 2
    up = (2 if c.activation == "swiglu" else 1) * c.intermediate_dim
    per_block = (P * hd + (c.num_heads if e.per_token_beta else 0)) * c.hidden_dim \
        + c.hidden_dim * hd + up * c.hidden_dim + c.hidden_dim * c.intermediate_dim
    mat = c.num_layers * per_block + c.vocab_size * c.hidden_dim
    efla = c.num_layers * c.num_heads * (4 * c.head_dim * c.head_dim + 8 * 64 * c.head_dim)
    return 6.0 * mat + 3.0 * efla


# ---- one block's tensors under the reference's names (shared with the pipeline stages) ----
def _put(dst, src):
    dst.copy_(src.to(dst.device, dst.dtype))


def block_reference_tensors(b: Block, p: str, cfg: ModelConfig, out: dict) -> dict:
    """Adds block ``b``'s tensors to ``out`` under prefix ``p`` (``blocks.{i}.``), reference
    names and (in, out) orientation (src/model/model.zig:494-521)."""
    hd = cfg.num_heads * cfg.head_dim
    out[p + "ln1.weight"] = b.ln1.weight.detach()
    if b.ln1.bias is not None:
        out[p + "ln1.bias"] = b.ln1.bias.detach()
    names = ["w_q", "w_k", "w_v"] if b.efla.P == 3 else ["w_k", "w_v"]
    parts = b.efla.w_qkv.detach()[:len(names) * hd].split(hd, dim=0)
    for nme, w in zip(names, parts):
        out[p + "efla." + nme] = w.t().contiguous()
    out[p + "efla.w_o"] = b.efla.w_o.detach().t().contiguous()
    if b.efla.per_token_beta:
        nb = len(names) * hd
        out[p + "efla.w_beta"] = b.efla.w_qkv.detach()[nb:nb + b.efla.H].t().contiguous()
    else:
        out[p + "efla.beta_param"] = b.efla.beta_param.detach()
    if b.prism is not None:
        for nme, t in b.prism.reference_tensors().items():
            out[p + "prism." + nme] = t
    out[p + "ln2.weight"] = b.ln2.weight.detach()
    if b.ln2.bias is not None:
        out[p + "ln2.bias"] = b.ln2.bias.detach()
    if b.mlp.act == "swiglu":
        g, u = b.mlp.gate_up_weights()
        out[p + "mlp_gate.weight"] = g.detach().t().contiguous()
        out[p + "mlp_up.weight"] = u.detach().t().contiguous()
    else:
        out[p + "mlp_up.weight"] = b.mlp.w_up.detach().t().contiguous()
    out[p + "mlp_down.weight"] = b.mlp.w_down.detach().t().contiguous()
    return out


@torch.no_grad()
def load_block_reference(b: Block, p: str, cfg: ModelConfig, tensors: dict) -> None:
    """Inverse of ``block_reference_tensors``."""
    hd = cfg.num_heads * cfg.head_dim
    _put(b.ln1.weight, tensors[p + "ln1.weight"])
    if b.ln1.bias is not None:
        _put(b.ln1.bias, tensors[p + "ln1.bias"])
    names = ["w_q", "w_k", "w_v"] if b.efla.P == 3 else ["w_k", "w_v"]
    for j, nme in enumerate(names):
        _put(b.efla.w_qkv[j * hd:(j + 1) * hd], tensors[p + "efla." + nme].t())
    _put(b.efla.w_o, tensors[p + "efla.w_o"].t())
    if b.efla.per_token_beta:
        nb = len(names) * hd
        _put(b.efla.w_qkv[nb:nb + b.efla.H], tensors[p + "efla.w_beta"].t())
    else:
        _put(b.efla.beta_param, tensors[p + "efla.beta_param"].reshape(1))
    if b.prism is not None:
        b.prism.load_reference_tensors({k[len(p + "prism."):]: v for k, v in tensors.items()
                                        if k.startswith(p + "prism.")})
    _put(b.ln2.weight, tensors[p + "ln2.weight"])
    if b.ln2.bias is not None:
        _put(b.ln2.bias, tensors[p + "ln2.bias"])
    if b.mlp.act == "swiglu":
        g, u = b.mlp.gate_up_weights()
        _put(g, tensors[p + "mlp_gate.weight"].t())
        _put(u, tensors[p + "mlp_up.weight"].t())
    else:
        _put(b.mlp.w_up, tensors[p + "mlp_up.weight"].t())
    _put(b.mlp.w_down, tensors[p + "mlp_down.weight"].t())
