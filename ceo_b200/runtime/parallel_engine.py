"""Training engine for tensor- and context-parallel runs: builds the device mesh from the
``runtime`` section of the config (``tensor_parallel_size``, ``context_parallel_size``, the
rest is data parallel; rank order pp -> dp -> tp -> cp innermost as in the reference's
``ParallelConfig.globalRank``, src/tensor/sharding.zig:401-412), the peer-memory contexts of
each group, the parallel model, and the sharded optimizer over the ranks that hold the same
parameter shard (data-parallel x context-parallel).

One step = micro-batched forward/backward -> sum of replicated-parameter gradients over the
tensor-parallel group -> fused reduce-scatter + AdamW + all-gather over the replica group.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.parallel_model import ParallelEflaLM, sync_replicated_grads
from ..optim.flat import FlatParams
from ..optim.optimizers import LRScheduler, build_optimizer
from ..parallel.comm import Comm
from ..parallel.sharding import ParallelConfig
from ..utils.config import Config


def _group_for(ranks, all_groups_ranks):
    """new_group is collective: every rank creates every group, keeps its own."""
    mine = None
    me = dist.get_rank()
    for rk in all_groups_ranks:
        g = dist.new_group(list(rk)) if len(rk) > 1 else None
        if me in rk:
            mine = g
    return mine


class ParallelEngine:
    def __init__(self, cfg: Config, device, fused: bool = True, impl: str | None = None):
        self.cfg = cfg
        self.device = torch.device(device)
        rt = cfg.runtime
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        tp, cp = rt.tensor_parallel_size, rt.context_parallel_size
        if world % (tp * cp):
            raise ValueError(f"world {world} is not a multiple of tp*cp = {tp * cp}")
        dp = world // (tp * cp)
        self.pc = ParallelConfig.from_global_rank(rank, 1, dp, tp, cp, rt.zero_stage)
        pcs = [ParallelConfig.from_global_rank(r, 1, dp, tp, cp) for r in range(world)]
        tp_sets = sorted({tuple(p.group_ranks("tp")) for p in pcs})
        cp_sets = sorted({tuple(p.group_ranks("sp")) for p in pcs})
        rep_sets = sorted({tuple(sorted(q.global_rank() for q in pcs if q.tp_rank == p.tp_rank))
                           for p in pcs})
        self.tp_group = _group_for(None, tp_sets) if world > 1 else None
        self.cp_group = _group_for(None, cp_sets) if world > 1 else None
        self.rep_group = _group_for(None, rep_sets) if world > 1 else None
        self.tp_size, self.cp_size, self.dp_size = tp, cp, dp
        self.rank, self.world = rank, world
        self.fp8 = None
        if cfg.training.fp8_training and rank == 0:
            import warnings
            warnings.warn("training.fp8_training is ignored by the tensor / context parallel "
                          "engine: its projections run in bf16", stacklevel=2)

        def make_comm(group, size):
            if size == 1:
                return None
            if fused:
                from ..parallel.fused import FusedComm
                return FusedComm(group)
            return Comm(group)
        self.tp_comm = make_comm(self.tp_group, tp)
        self.cp_comm = make_comm(self.cp_group, cp)
        self.rep_comm = make_comm(self.rep_group, dp * cp)
        self.impl = impl or ("fused" if fused else "nccl")
        m = cfg.model
        self.micro_batch = cfg.training.micro_batch_size
        seq_local = cfg.data.seq_len // cp
        self.tp_ctx = self.cp_ctx = None
        if tp > 1:
            from ..parallel.tp import TPContext
            if not fused:
                raise ValueError("tensor parallelism needs the peer-memory contexts (fused=True); "
                                 "impl='nccl' then selects the NCCL compositions on top of them")
            rows = self.micro_batch * seq_local
            widest = max(m.hidden_dim, 3 * m.num_heads * m.head_dim // tp,
                         2 * m.intermediate_dim // tp)
            self.tp_ctx = TPContext(self.tp_comm, rows, widest)
        if cp > 1:
            from ..parallel.cp import CPContext
            self.cp_ctx = CPContext(self.cp_comm, self.micro_batch * m.num_heads // tp, m.head_dim)
        self.model = ParallelEflaLM(m, self.device, self.tp_ctx, self.cp_ctx, seed=rt.seed,
                                    impl=self.impl)
        rep_world = dp * cp
        rep_rank = dist.get_rank(self.rep_group) if self.rep_group is not None else 0
        self.flat = FlatParams(self.model, rep_world, rep_rank,
                               alloc=getattr(self.rep_comm, "alloc", None))
        self.optimizer = build_optimizer(self.flat, cfg.training, self.rep_comm)
        if tp > 1:
            # the gradient norm spans the tensor-parallel group; replicated tensors count once
            self.optimizer.extra_norm_group = self.tp_group
            self.optimizer.replicated_names = {n for n, p in self.model.named_parameters()
                                               if getattr(p, "replicated", False)}
            self.optimizer.use_fused_step = False
        t = cfg.training
        self.scheduler = LRScheduler(t.learning_rate, t.min_learning_rate, t.warmup_steps,
                                     t.total_steps, t.lr_schedule)
        self.step_count = 0
        self.tokens_seen = 0
        self.cp_rank = self.pc.sp_rank
        self.zero_stage = 1 if rep_world > 1 else 0

    def materialize_params(self):
        pass

    def local_span(self, tokens: torch.Tensor) -> torch.Tensor:
        """This rank's contiguous span of the sequence dimension under context parallelism."""
        if self.cp_size == 1:
            return tokens
        T = tokens.shape[1] // self.cp_size
        if tokens.shape[1] % self.cp_size or T % 64:
            # the state crosses ranks at chunk boundaries: every span is whole 64-token chunks
            raise ValueError(f"sequence length {tokens.shape[1]} does not split into "
                             f"{self.cp_size} context-parallel spans of whole 64-token chunks")
        return tokens[:, self.cp_rank * T:(self.cp_rank + 1) * T].contiguous()

    def train_step(self, batches, lr: float | None = None):
        """``batches``: list of (tokens, targets), each the (micro_batch, seq_len) batch of this
        rank's data-parallel replica (identical on the ranks of one tp x cp group)."""
        n = len(batches)
        if lr is None:
            lr = self.scheduler.get_lr()
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        for tok, tgt, *_ in batches:
            tok = self.local_span(tok.to(self.device, non_blocking=True))
            tgt = self.local_span(tgt.to(self.device, non_blocking=True))
            loss = self.model(tok, tgt, self.cfg.training.label_smoothing)
            loss.backward()
            total += loss.detach().float()
            self.tokens_seen += tok.numel() * self.cp_size * self.dp_size
        sync_replicated_grads(self.model, self.tp_group)
        scale = 1.0 / (n * self.tp_size * self.cp_size * self.dp_size)
        gnorm = self.optimizer.step(lr, grad_scale=scale)
        self.scheduler.step()
        self.step_count += 1
        mean = total / n
        if self.world > 1:
            dist.all_reduce(mean)
            mean = mean / self.world
        return mean, gnorm

    def close(self):
        for c in (self.tp_ctx, self.cp_ctx):
            if c is not None:
                c.close()
        for c in (self.tp_comm, self.cp_comm, self.rep_comm):
            if c is not None and hasattr(c, "close"):
                c.close()


class PipelineEngine:
    """Training engine for pipeline-parallel runs (``runtime.pipeline_parallel_size`` > 1):
    the blocks are cut into contiguous stages (``parallel.pipeline``), micro-batches flow
    through them on the 1F1B schedule with point-to-point exchanges of the library, and the
    ranks that hold the same stage (the data-parallel group) share a sharded optimizer.
    Rank order pp -> dp as in the reference's ``ParallelConfig.globalRank``
    (src/tensor/sharding.zig:401-412).  Tensor and context parallelism inside a stage are not
    combined with it."""

    def __init__(self, cfg: Config, device):
        from ..parallel.pipeline import PipelineRunner, PipelineStage
        self.cfg = cfg
        self.device = torch.device(device)
        rt = cfg.runtime
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        pp = rt.pipeline_parallel_size
        if rt.tensor_parallel_size * rt.context_parallel_size != 1:
            raise ValueError("pipeline parallelism is not combined with tensor / context "
                             "parallelism: set tensor_parallel_size = context_parallel_size = 1")
        if world % pp:
            raise ValueError(f"world {world} is not a multiple of the pipeline size {pp}")
        dp = world // pp
        self.pc = ParallelConfig.from_global_rank(rank, pp, dp, 1, 1, rt.zero_stage)
        pcs = [ParallelConfig.from_global_rank(r, pp, dp, 1, 1) for r in range(world)]
        pp_sets = sorted({tuple(p.group_ranks("pp")) for p in pcs})
        dp_sets = sorted({tuple(p.group_ranks("dp")) for p in pcs})
        self.pp_group = _group_for(None, pp_sets) if world > 1 else None
        self.dp_group = _group_for(None, dp_sets) if world > 1 else None
        self.pp_size, self.dp_size, self.tp_size, self.cp_size = pp, dp, 1, 1
        self.rank, self.world = rank, world
        self.fp8 = None
        self.zero_stage = 1 if dp > 1 else 0
        dtype = torch.bfloat16 if self.device.type == "cuda" else None
        self.model = PipelineStage(cfg.model, self.device, self.pc.pp_rank, pp, seed=rt.seed,
                                   dtype=dtype)
        self.runner = PipelineRunner(self.model, self.pp_group)
        self.dp_comm = Comm(self.dp_group) if dp > 1 else None
        self.flat = FlatParams(self.model, dp, self.pc.dp_rank)
        self.optimizer = build_optimizer(self.flat, cfg.training, self.dp_comm)
        if pp > 1:
            self.optimizer.extra_norm_group = self.pp_group  # the norm spans all stages
            self.optimizer.use_fused_step = False
        t = cfg.training
        self.scheduler = LRScheduler(t.learning_rate, t.min_learning_rate, t.warmup_steps,
                                     t.total_steps, t.lr_schedule)
        self.step_count = 0
        self.tokens_seen = 0

    def train_step(self, batches, lr: float | None = None):
        """``batches``: this data-parallel replica's micro-batches (the same list on every
        stage of the replica)."""
        n = len(batches)
        if lr is None:
            lr = self.scheduler.get_lr()
        dev_batches = [tuple(x.to(self.device, non_blocking=True) for x in b[:2]) for b in batches]
        loss = self.runner.run(dev_batches, self.cfg.training.label_smoothing, scale_loss=False)
        self.runner.sync_tied_grads()
        for tok, _ in dev_batches:
            self.tokens_seen += tok.numel() * self.dp_size
        gnorm = self.optimizer.step(lr, grad_scale=1.0 / (n * self.dp_size))
        self.scheduler.step()
        self.step_count += 1
        if self.dp_comm is not None:
            self.dp_comm.all_reduce(loss)
            loss = loss / self.dp_size
        return loss, gnorm

    def materialize_params(self):
        pass

    def close(self):
        pass


def build_engine(cfg: Config, device, comm=None):
    """The engine the ``runtime`` section asks for: pipeline stages when
    ``pipeline_parallel_size`` > 1, the tensor / context parallel engine when
    ``tensor_parallel_size x context_parallel_size`` > 1, else the data-parallel
    ``TrainEngine`` (ZeRO stage from ``zero_stage``) on ``comm``."""
    rt = cfg.runtime
    if rt.pipeline_parallel_size > 1:
        return PipelineEngine(cfg, device)
    if rt.tensor_parallel_size * rt.context_parallel_size > 1:
        return ParallelEngine(cfg, device)
    from .engine import TrainEngine
    return TrainEngine(cfg, device, comm)
