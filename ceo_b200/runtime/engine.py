"""The training step: micro-batched forward/backward with gradients accumulated in fp32
by the GEMM epilogues, then one sharded optimizer step.

This is the hot loop the reference's Trainer only sketches (forwardStep / backwardStep /
updateStep in src/runtime/trainer.zig:245-308 run a CPU-only forward, a stub backward and
a constant loss).  Inputs arrive as pinned host tensors and are copied to the device
asynchronously one micro-batch ahead of the compute.
"""
from __future__ import annotations

import torch

from ..utils.tracing import trace_range

from ..models.model import EflaLM
from ..optim.flat import FlatParams
from ..optim.optimizers import LRScheduler, build_optimizer
from ..utils.config import Config


class TrainEngine:
    def __init__(self, cfg: Config, device, comm=None, seed: int | None = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        seed = cfg.runtime.seed if seed is None else seed
        dtype = None
        if self.device.type == "cuda":
            dtype = torch.bfloat16
        if self.device.type == "cuda":
            from ..ops import _lib
            _lib.lib().ceo_set_deterministic(int(cfg.runtime.deterministic))
        self.model = EflaLM(cfg.model, self.device, dtype=dtype, seed=seed)
        # training.fp8_training (src/util/config.zig:420): forward projections on e4m3 operands
        g8 = bool(getattr(cfg.training, "fp8_gradients", False))
        # two bits of headroom above the recorded amax: with margin 0 the delayed scales clip
        # while activations and gradients still grow quickly (first steps of a run)
        self.fp8 = self.model.enable_fp8(margin=2, dgrad=g8, wgrad=g8) \
            if cfg.training.fp8_training else None
        # ZeRO stage (runtime.zero_stage): with the peer-memory communicator and AdamW / Lion
        # the flat buffers use the row-sharded segment layout and stage 1, 2 or 3 as configured
        # (parallel/fsdp.py); every other combination shards the optimizer state over
        # contiguous slices with library collectives (stage 1 semantics).
        fused = (self.world > 1 and getattr(comm, "fused", False)
                 and cfg.training.optimizer in ("adamw", "lion") and self.device.type == "cuda"
                 and self.world in (2, 4, 8))
        stage = int(cfg.runtime.zero_stage)
        self.zero_stage = 0 if self.world == 1 else (max(1, min(3, stage)) if fused else 1)
        self.flat = FlatParams(self.model, self.world, self.rank,
                               alloc=getattr(comm, "alloc", None),
                               layout="segment" if fused else "contiguous")
        self.optimizer = build_optimizer(self.flat, cfg.training, comm)
        self.reducer = None
        self.gathers = []
        if fused and self.zero_stage >= 2:
            from ..parallel.fsdp import BucketReducer
            self.reducer = BucketReducer(comm, self.flat,
                                         [f"blocks.{i}." for i in range(len(self.model.blocks))])
            self.model.block_input_hook = self.reducer.block_hook
        if fused and self.zero_stage >= 3:
            if self.fp8 is not None:
                raise ValueError("runtime.zero_stage 3 and training.fp8_training cannot be "
                                 "combined: the fused weight gather is a bf16 GEMM")
            from ..parallel.fsdp import attach_weight_gathers
            self.gathers = attach_weight_gathers(self.model, comm, self.flat)
        t = cfg.training
        self.scheduler = LRScheduler(t.learning_rate, t.min_learning_rate, t.warmup_steps,
                                     t.total_steps, t.lr_schedule)
        self.label_smoothing = t.label_smoothing
        self.step_count = 0
        self.tokens_seen = 0
        self._copy_stream = torch.cuda.Stream() if self.device.type == "cuda" else None

    # ------------------------------------------------------------------------------
    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device:
            return t
        return t.to(self.device, non_blocking=True)

    def train_step(self, batches, lr: float | None = None):
        """``batches``: a list (one entry per micro-batch) of (tokens, targets) integer tensors
        of shape (mb, T), on the host (pinned) or already on the device; an optional third
        entry ``resets`` (mb, T/64, bool) marks the chunks that start a new document of a
        packed batch (``data.dataset.packed_batch``).
        Returns (mean loss, gradient norm) as device scalars."""
        n = len(batches)
        if lr is None:
            lr = self.scheduler.get_lr()
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        nxt = None
        if self._copy_stream is not None:
            with torch.cuda.stream(self._copy_stream):
                nxt = tuple(self._to_device(x) for x in batches[0])
        for i in range(n):
            if self._copy_stream is not None:
                torch.cuda.current_stream().wait_stream(self._copy_stream)
                tok, tgt, *rest = nxt
                for x in nxt:
                    x.record_stream(torch.cuda.current_stream())
                if i + 1 < n:
                    with torch.cuda.stream(self._copy_stream):
                        nxt = tuple(self._to_device(x) for x in batches[i + 1])
            else:
                tok, tgt, *rest = batches[i]
            resets = rest[0] if rest else None
            with trace_range("forward"):
                loss = self.model(tok, tgt, self.label_smoothing, resets=resets)
            if self.reducer is not None and i == n - 1:
                # last micro-batch: each block's gradients leave for their owners as soon as
                # the block's backward is done
                self.reducer.armed = True
            with trace_range("backward"):
                loss.backward()
            total += loss.detach().float()
            self.tokens_seen += tok.numel() * self.world
        # mean over micro-batches and data-parallel ranks (the collectives sum)
        with trace_range("optimizer"):
            if self.reducer is not None:
                self.reducer.finish()
                self.optimizer.grads_reduced = True
            gnorm = self.optimizer.step(lr, grad_scale=1.0 / (n * self.world))
            for g in self.gathers:
                g.pending = True
        if self.fp8 is not None:
            self.fp8.step()
        self.scheduler.step()
        self.step_count += 1
        mean = total / n
        if self.comm is not None and self.world > 1:
            self.comm.all_reduce(mean)
            mean = mean / self.world
        return mean, gnorm

    def materialize_params(self):
        """ZeRO stage 3: completes every rank's local copy of the parameters that the last
        optimizer step left as row shards (a collective: every rank must call it).  Needed
        before reading parameters outside a training step (checkpoints, evaluation)."""
        for g in self.gathers:
            g.materialize()

    @torch.no_grad()
    def eval_loss(self, tok, tgt):
        self.materialize_params()
        return self.model(self._to_device(tok), self._to_device(tgt))
