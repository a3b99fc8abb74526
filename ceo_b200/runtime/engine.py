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
        self.flat = FlatParams(self.model, self.world, self.rank,
                               alloc=getattr(comm, "alloc", None))
        self.optimizer = build_optimizer(self.flat, cfg.training, comm)
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
        of shape (mb, T), on the host (pinned) or already on the device.
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
                tok, tgt = nxt
                tok.record_stream(torch.cuda.current_stream())
                tgt.record_stream(torch.cuda.current_stream())
                if i + 1 < n:
                    with torch.cuda.stream(self._copy_stream):
                        nxt = tuple(self._to_device(x) for x in batches[i + 1])
            else:
                tok, tgt = batches[i]
            with trace_range("forward"):
                loss = self.model(tok, tgt, self.label_smoothing)
            with trace_range("backward"):
                loss.backward()
            total += loss.detach().float()
            self.tokens_seen += tok.numel() * self.world
        # mean over micro-batches and data-parallel ranks (the collectives sum)
        with trace_range("optimizer"):
            gnorm = self.optimizer.step(lr, grad_scale=1.0 / (n * self.world))
        if self.fp8 is not None:
            self.fp8.step()
        self.scheduler.step()
        self.step_count += 1
        mean = total / n
        if self.comm is not None and self.world > 1:
            self.comm.all_reduce(mean)
            mean = mean / self.world
        return mean, gnorm

    @torch.no_grad()
    def eval_loss(self, tok, tgt):
        return self.model(self._to_device(tok), self._to_device(tgt))
