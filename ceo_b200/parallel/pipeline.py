"""Pipeline parallelism: the blocks of an ``EflaLM`` are cut into contiguous stages, one per
rank of the pipeline group, and micro-batches flow through them on the one-forward-one-
backward schedule (warm-up forwards, steady 1F1B, cool-down backwards), activations and their
gradients moving between neighbours with point-to-point sends.

The reference only describes this axis: ``pp_world_size`` / ``pp_rank`` and the rank order
pp -> dp -> tp -> sp (src/tensor/sharding.zig:362-363, 401-412), ``pipeline_parallel_size``
(src/util/config.zig:489) and ``ncclSend`` / ``ncclRecv`` wrappers (src/runtime/nccl.zig:
308-331); both of its configs set the size to 1.

Weights are the ones the single-process model draws from the same seed, so a pipeline and the
whole model are the same function.  With tied embeddings the last stage keeps its own copy of
the embedding for the LM head; ``sync_tied_grads`` sums the two copies' gradients.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.model import EflaLM
from ..ops import nn as K
from ..utils.config import ModelConfig


def stage_bounds(num_layers: int, stages: int, stage: int) -> tuple[int, int]:
    """Layers [lo, hi) of a stage; the first ``num_layers % stages`` stages take one more."""
    base, rem = divmod(num_layers, stages)
    lo = stage * base + min(stage, rem)
    return lo, lo + base + (1 if stage < rem else 0)


class PipelineStage(nn.Module):
    """The slice of the model one pipeline rank runs."""

    def flops_per_token(self, seq_len=None) -> float:
        """Of the WHOLE model (all stages), for throughput accounting."""
        from ..models.model import model_flops_per_token
        return model_flops_per_token(self.cfg)

    def count_parameters(self) -> int:
        """Parameters this stage holds."""
        return sum(p.numel() for p in self.parameters())

    def state_dict_shards(self):
        """name -> (tensor, None): this stage's tensors under the reference's names."""
        from ..models.model import block_reference_tensors
        out = {}
        if self.first:
            out["embed_tokens.weight"] = self.embed_tokens.detach()
        for j, b in enumerate(self.blocks):
            block_reference_tensors(b, f"blocks.{self.lo + j}.", self.cfg, out)
        if self.last:
            out["final_norm.weight"] = self.final_norm.weight.detach()
            if self.final_norm.bias is not None:
                out["final_norm.bias"] = self.final_norm.bias.detach()
            if self.lm_head is not None:
                out["lm_head.weight"] = self.lm_head.detach().t().contiguous()
        return {k: (v, None) for k, v in out.items()}

    @torch.no_grad()
    def load_reference_state(self, tensors: dict) -> None:
        """Keeps this stage's part of a FULL set of tensors (reference names)."""
        from ..models.model import _put, load_block_reference
        if self.embed_tokens is not None:
            _put(self.embed_tokens, tensors["embed_tokens.weight"])
        for j, b in enumerate(self.blocks):
            load_block_reference(b, f"blocks.{self.lo + j}.", self.cfg, tensors)
        if self.last:
            _put(self.final_norm.weight, tensors["final_norm.weight"])
            if self.final_norm.bias is not None:
                _put(self.final_norm.bias, tensors["final_norm.bias"])
            if self.lm_head is not None:
                _put(self.lm_head, tensors["lm_head.weight"].t())

    def __init__(self, cfg: ModelConfig, device, stage: int, stages: int, seed: int = 0,
                 dtype=None):
        super().__init__()
        full = EflaLM(cfg, device, dtype=dtype, seed=seed)
        self.cfg, self.stage, self.stages = cfg, stage, stages
        self.first, self.last = stage == 0, stage == stages - 1
        self.lo, self.hi = stage_bounds(cfg.num_layers, stages, stage)
        self.blocks = nn.ModuleList(full.blocks[self.lo:self.hi])
        self.embed_tokens = full.embed_tokens if (self.first or (self.last and cfg.tie_embeddings)) \
            else None
        self.final_norm = full.final_norm if self.last else None
        self.lm_head = full.lm_head if (self.last and not cfg.tie_embeddings) else None
        self.act_dtype = full.embed_tokens.dtype
        del full

    def forward(self, x, targets=None, label_smoothing: float = 0.0):
        """First stage: x = tokens (B,T).  Others: x = hidden states (B,T,D).  The last stage
        returns the mean loss, every other one the hidden states for its successor."""
        h = K.embedding(x, self.embed_tokens) if self.first else x
        for blk in self.blocks:
            h, _ = blk(h)
        if not self.last:
            return h
        hn = self.final_norm(h)
        w = self.embed_tokens if self.lm_head is None else self.lm_head
        return K.linear_cross_entropy(hn, w, targets, label_smoothing)


def _p2p(ops):
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()


class PipelineRunner:
    """Runs one optimizer step's micro-batches through a stage on the 1F1B schedule."""

    def __init__(self, stage: PipelineStage, group=None):
        self.stage, self.group = stage, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert self.world == stage.stages and self.rank == stage.stage
        g = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
        self.prev = g(self.rank - 1) if self.rank > 0 else None
        self.next = g(self.rank + 1) if self.rank < self.world - 1 else None
        self.first_global, self.last_global = g(0), g(self.world - 1)

    # -- neighbour exchanges (a send and a receive that face each other go out as one batch,
    #    so two stages never block on each other's send) ---------------------------------------
    def _exchange(self, send_t, send_to, recv_shape, recv_from, dtype, device):
        ops, got = [], None
        if send_t is not None and send_to is not None:
            ops.append(dist.P2POp(dist.isend, send_t.contiguous(), send_to, self.group))
        if recv_shape is not None and recv_from is not None:
            got = torch.empty(recv_shape, dtype=dtype, device=device)
            ops.append(dist.P2POp(dist.irecv, got, recv_from, self.group))
        _p2p(ops)
        return got

    def run(self, batches, label_smoothing: float = 0.0, scale_loss: bool = True) -> torch.Tensor:
        """``batches``: list of (tokens, targets), the same on every stage.  Gradients
        accumulate in the parameters: their mean over the micro-batches, or, with
        ``scale_loss=False``, their SUM (every loss back-propagated with gradient 1, which is
        what the fp32 ``main_grad`` accumulation of the GEMM epilogues assumes; the caller
        then folds 1/n into the optimizer's gradient scale).  Returns the mean loss (valid on
        every rank: the last stage broadcasts it)."""
        n = len(batches)
        st = self.stage
        dev = batches[0][0].device
        hshape = (*batches[0][0].shape, st.cfg.hidden_dim)
        dt = st.act_dtype
        warm = min(self.world - 1 - self.rank, n)
        steady = n - warm
        pending = []
        total = torch.zeros((), dtype=torch.float32, device=dev)
        fwd_i = 0

        def forward(x_in):
            nonlocal fwd_i, total
            tok, tgt = batches[fwd_i]
            fwd_i += 1
            x = tok if st.first else x_in.requires_grad_(True)
            out = st(x, tgt, label_smoothing)
            if st.last:
                total += out.detach().float()
            pending.append((x, out))
            return out

        def backward(g):
            x, out = pending.pop(0)
            if st.last:
                (out / n if scale_loss else out).backward()
            else:
                torch.autograd.backward(out, grad_tensors=g)
            return None if st.first else x.grad

        recv_fwd = lambda: self._exchange(None, None, hshape, self.prev, dt, dev)  # noqa: E731
        for _ in range(warm):
            out = forward(recv_fwd())
            self._exchange(out.detach() if not st.last else None, self.next, None, None, dt, dev)
        x_in = recv_fwd() if steady > 0 else None
        for i in range(steady):
            out = forward(x_in)
            g = self._exchange(None if st.last else out.detach(), self.next,
                               None if st.last else hshape, self.next, dt, dev)
            dx = backward(g)
            x_in = self._exchange(dx, self.prev, hshape if i + 1 < steady else None, self.prev, dt,
                                  dev)
        for _ in range(warm):
            g = self._exchange(None, None, None if st.last else hshape, self.next, dt, dev)
            dx = backward(g)
            self._exchange(dx, self.prev, None, None, dt, dev)
        total = total / n
        if self.world > 1:
            dist.broadcast(total, src=self.last_global, group=self.group)
        return total

    def sync_tied_grads(self):
        """Sums the embedding gradient of the first stage and of the last stage's head copy."""
        st = self.stage
        if not st.cfg.tie_embeddings or self.world == 1 or not (st.first or st.last):
            return
        p = st.embed_tokens
        g = getattr(p, "main_grad", None)
        if g is None:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            g = p.grad
        peer = self.last_global if st.first else self.first_global
        other = torch.empty_like(g)
        ops = [dist.P2POp(dist.isend, g.contiguous(), peer, self.group),
               dist.P2POp(dist.irecv, other, peer, self.group)]
        _p2p(ops)
        g.add_(other)
