"""Trainer: config -> engine -> data -> loop with logging, checkpointing and resume.

Public surface of the reference's Trainer (src/runtime/trainer.zig): ``init`` (38-115),
``run`` (124-188), ``smoke_test`` (191-223: 3 iterations, B=1, T=16), ``resume`` (226-242),
``save_checkpoint`` (331-362).  Where the reference logs a constant loss of 10.0
(trainer.zig:269-272), passes the parameters as gradients (src/model/model.zig:527-529) and
never saves optimizer or RNG state (trainer.zig:356-357), this one trains: the loss is the
model's cross-entropy, checkpoints carry fp32 master weights, moments, RNG, the loader cursor
and the scheduler step, and ``resume`` restores all of them.
"""
from __future__ import annotations

import math
import os
import time

import torch

from ..data.dataset import (BinaryDataset, DataLoader, Prefetcher, pack_sequences,
                            packed_batch)
from ..data.synthetic import SyntheticTokens
from ..utils import errors
from ..utils.config import Config
from ..utils.telemetry import HealthStatus, Telemetry
from .checkpoint import CheckpointManager
from .engine import TrainEngine
from .fault import Heartbeat, KernelWatch, StepGuard


def _git_revision() -> str:
    try:
        import subprocess
        r = subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5,
                           cwd=os.path.dirname(os.path.abspath(__file__)))
        rev = r.stdout.strip()
        return rev if len(rev) == 40 else "0" * 40
    except Exception:  # noqa: BLE001
        return "0" * 40


class Trainer:
    def __init__(self, cfg: Config, device=None, comm=None, telemetry: Telemetry | None = None,
                 data_path: str | None = None, checkpoint_dir: str | None = None):
        self.cfg = cfg
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.comm = comm
        import torch.distributed as dist
        if comm is not None:
            self.rank, self.world = comm.rank, comm.world
        elif dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(), dist.get_world_size()
        else:
            self.rank, self.world = 0, 1
        # runtime.{tensor,context,pipeline}_parallel_size pick the engine
        # (src/util/config.zig:487-489,509-510; rank order src/tensor/sharding.zig:357-421)
        from .parallel_engine import build_engine
        self.engine = build_engine(cfg, self.device, comm)
        rt = cfg.runtime
        self.model_parallel = rt.tensor_parallel_size * rt.context_parallel_size * \
            rt.pipeline_parallel_size
        if self.model_parallel > 1:
            pc = self.engine.pc
            self.dp_rank, self.dp_world = pc.dp_rank, pc.dp_world_size
        else:
            self.dp_rank, self.dp_world = self.rank, self.world
        self.telemetry = telemetry or Telemetry(rank=self.rank, log_file=None,
                                                log_level=cfg.telemetry.log_level)
        if self.engine.fp8 is not None:
            self.telemetry.log("info", "trainer", "FP8 forward projections enabled "
                               f"({len(self.engine.fp8.states)} linears, delayed scaling, "
                               f"history {self.engine.fp8.history})")
        ck = cfg.checkpoint
        self.ckpt = CheckpointManager(checkpoint_dir or ck.dir, ck.keep_last_n, ck.save_optimizer,
                                      ck.async_save, self.rank, self.world)
        self.data_path = data_path or cfg.data.path
        # Failure detection: the device status word (a bounded wait in a kernel ran out) is
        # read every metrics interval and before every checkpoint; with more than one rank a
        # store heartbeat is consulted before each step, so a dead peer is noticed on the host
        # before the next kernel that would wait for it is launched.
        self.guard = self._make_guard()
        self.loader = None
        self._prefetch = None
        self._packing = False
        self.epoch = 0
        self.last_loss = float("nan")
        t = cfg.training
        dp = max(1, self.dp_world)
        self.micro_batch = t.micro_batch_size
        self.n_micro = max(1, t.global_batch_size // (t.micro_batch_size * dp))
        # training.gradient_accumulation_steps (src/util/config.zig:407) must agree with
        # global / (micro x data-parallel ranks), which is what the step runs
        gas = int(getattr(t, "gradient_accumulation_steps", 0) or 0)
        if gas not in (0, self.n_micro):
            self.telemetry.log("warn", "config", f"gradient_accumulation_steps = {gas} does not "
                               f"match global_batch_size / (micro_batch_size x {dp} ranks) = "
                               f"{self.n_micro}; running {self.n_micro} micro-batches per step")

    def _make_guard(self) -> StepGuard:
        kw = KernelWatch() if self.device.type == "cuda" else None
        hb = None
        if self.world > 1:
            try:
                import torch.distributed as dist
                from torch.distributed.distributed_c10d import _get_default_store
                if dist.is_initialized():
                    hb = Heartbeat(_get_default_store(), self.rank, self.world, interval=2.0,
                                   timeout=120.0).start()
            except Exception as e:  # noqa: BLE001  (no store: status-word checks only)
                self.telemetry.log("warn", "trainer", f"heartbeat unavailable: {e}")
        return StepGuard(hb, kw, check_every=max(1, self.cfg.telemetry.metrics_interval))

    # ------------------------------------------------------------------------- data
    def _open_data(self):
        d = self.cfg.data
        if d.synthetic.kind:
            self._synth = SyntheticTokens(self.cfg.model.vocab_size, d.synthetic.kind,
                                          d.synthetic.s, d.synthetic.seed, self.dp_rank)
            return
        self._synth = None
        ds = BinaryDataset.open(self.data_path)
        self.loader = DataLoader(ds, d.seq_len, self.micro_batch, shuffle=True, drop_last=True,
                                 seed=self.cfg.runtime.seed, dp_rank=self.dp_rank,
                                 dp_world=self.dp_world, pin=self.device.type == "cuda")
        if len(self.loader) == 0:
            raise errors.DataExhausted(
                f"{self.data_path}: not enough tokens for one batch of {self.micro_batch} x "
                f"{d.seq_len + 1}")
        # data.pack_sequences (src/util/config.zig:567): windows are cut at the end-of-document
        # token and the documents packed on 64-token boundaries, with the recurrent state
        # reset at every document start; needs a sequence length that is a multiple of 64
        self._packing = bool(d.pack_sequences) and d.eos_token_id >= 0 and d.seq_len % 64 == 0
        self._packs = []

    def _loader_state(self):
        if self.loader is None:
            return None
        return self._prefetch.state_dict() if self._prefetch is not None else \
            self.loader.state_dict()

    def _close_data(self):
        if self._prefetch is not None:
            self._prefetch.close()
            self._prefetch = None

    def _next_window_batch(self):
        """The next (inputs, targets) window batch, read ``data.prefetch_factor`` batches ahead
        on a background thread (src/util/config.zig:565); rolls over to the next epoch."""
        while True:
            if self.cfg.data.prefetch_factor > 0:
                if self._prefetch is None:
                    self._prefetch = Prefetcher(self.loader, self.cfg.data.prefetch_factor)
                b = self._prefetch.next()
            else:
                b = self.loader.next()
            if b is not None:
                return b
            self._close_data()
            self.loader.reset()
            self.epoch += 1

    def _next_packed(self):
        """One packed micro-batch (tokens, targets, resets) of ``micro_batch`` rows."""
        d = self.cfg.data
        while len(self._packs) < self.micro_batch:
            b = self._next_window_batch()
            full = torch.cat([b.input, b.target[:, -1:]], dim=1).numpy()
            docs = []
            for row in full:
                cuts = (row == d.eos_token_id).nonzero()[0] + 1
                lo = 0
                for c in list(cuts) + [len(row)]:
                    if c > lo:
                        docs.append(row[lo:c])
                    lo = c
            self._packs += pack_sequences(docs, d.seq_len + 1, align=64)
        take, self._packs = self._packs[:self.micro_batch], self._packs[self.micro_batch:]
        tok, tgt, resets = packed_batch(take, 64)
        if self.device.type == "cuda":
            tok, tgt, resets = tok.pin_memory(), tgt.pin_memory(), resets.pin_memory()
        return tok, tgt, resets

    def _next_micro_batches(self):
        out = []
        if self._synth is not None:
            for _ in range(self.n_micro):
                out.append(self._synth.batch(self.micro_batch, self.cfg.data.seq_len,
                                             pin=self.device.type == "cuda"))
            return out
        while len(out) < self.n_micro:
            if self._packing:
                out.append(self._next_packed())
            else:
                b = self._next_window_batch()
                out.append((b.input, b.target))
        return out

    # ------------------------------------------------------------------------- loop
    def run(self, max_steps: int | None = None) -> dict:
        cfg, eng, tel = self.cfg, self.engine, self.telemetry
        self._open_data()
        total = cfg.training.total_steps if max_steps is None else \
            min(cfg.training.total_steps, eng.step_count + max_steps)
        tokens_per_step = self.micro_batch * self.n_micro * cfg.data.seq_len * self.dp_world
        flops_tok = eng.model.flops_per_token(cfg.data.seq_len)
        tel.log("info", "trainer", f"training {cfg.model.name}: {eng.model.count_parameters()} "
                f"parameters, {tokens_per_step} tokens/step, {self.world} rank(s)")
        use_events = self.device.type == "cuda"
        while eng.step_count < total:
            batches = self._next_micro_batches()
            lr = eng.scheduler.get_lr()
            if use_events:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            t0 = time.time()
            self.guard.before_step()
            loss, gnorm = eng.train_step(batches, lr)
            self.guard.after_step()  # status word every metrics interval (one host read)
            step = eng.step_count
            log_now = step % max(1, cfg.telemetry.metrics_interval) == 0 or step == total
            if log_now:
                if use_events:
                    e1.record()
                    e1.synchronize()
                    secs = e0.elapsed_time(e1) * 1e-3
                    if self.comm is not None:
                        secs = self.comm.max_over_ranks(secs)
                    elif self.world > 1:
                        import torch.distributed as dist
                        tmax = torch.tensor([secs], dtype=torch.float64, device=self.device)
                        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
                        secs = float(tmax)
                else:
                    secs = time.time() - t0
                lv, gv = float(loss), float(gnorm)
                self.last_loss = lv
                if not math.isfinite(lv):
                    tel.log_health_check(HealthStatus(nan_inf=True))
                    raise errors.NaNDetected(f"loss is {lv} at step {step}")
                tel.stats.update(lv, tokens_per_step, secs)
                tps = tokens_per_step / secs if secs > 0 else 0.0
                mfu = None
                if use_events:
                    from ..utils.kernel_bench import peaks
                    mfu = tps * flops_tok / self.world / peaks()[1]
                tel.log_step(step, eng.tokens_seen, lr, gv)
                tel.log_metrics(step, lv, lr, eng.tokens_seen, tps, mfu)
            if cfg.checkpoint.save_interval > 0 and step % cfg.checkpoint.save_interval == 0:
                self.save_checkpoint()
        self.ckpt.wait()
        self._close_data()
        if self.guard.hb is not None:
            self.guard.hb.stop()
        return {"step": eng.step_count, "loss": self.last_loss, "tokens_seen": eng.tokens_seen}

    def smoke_test(self, iterations: int = 3) -> list[float]:
        """3 optimizer steps on a B=1, T=16 batch (64 on a GPU, the kernels' chunk length)."""
        T = 16 if self.device.type != "cuda" else 64
        g = torch.Generator().manual_seed(self.cfg.runtime.seed)
        x = torch.randint(0, self.cfg.model.vocab_size, (1, T + 1), generator=g)
        losses = []
        for _ in range(iterations):
            loss, _ = self.engine.train_step([(x[:, :-1].contiguous(), x[:, 1:].contiguous())])
            losses.append(float(loss))
            self.telemetry.log("info", "smoke", f"iteration {len(losses)} loss {losses[-1]:.4f}")
        return losses

    # ------------------------------------------------------------------ checkpointing
    def save_checkpoint(self) -> str:
        eng = self.engine
        if self.guard.kw is not None:
            self.guard.kw.check()  # never checkpoint state a timed-out kernel may have left
        eng.materialize_params()  # ZeRO stage 3: complete the local parameter copy first
        md = {"step": eng.step_count, "epoch": self.epoch, "tokens_seen": eng.tokens_seen,
              "loss": self.last_loss if math.isfinite(self.last_loss) else 0.0,
              "learning_rate": eng.scheduler.get_lr(), "git_revision": _git_revision(),
              "config_hash": self.cfg.config_hash().hex()}
        opt = {"master": eng.flat.master}
        opt.update({k: v for k, v in eng.flat.state.items()})
        for name, st in eng.optimizer._muon_state.items():
            for k, v in st.items():
                opt[f"muon.{name}.{k}"] = v
        for name, st in eng.optimizer._side_state.items():
            for k, v in st.items():
                opt[f"side.{name}.{k}"] = v
        opt["step_count"] = torch.tensor([eng.optimizer.step_count], dtype=torch.int64)
        rng = torch.get_rng_state().numpy().tobytes()
        rt = self.cfg.runtime
        extra = {"scheduler": eng.scheduler.state_dict(),
                 "loader": self._loader_state(),
                 "flat_layout": eng.flat.layout_info(),
                 "mesh": {"pp": rt.pipeline_parallel_size, "tp": rt.tensor_parallel_size,
                          "cp": rt.context_parallel_size, "world": self.world}}
        if eng.fp8 is not None:
            extra["fp8"] = eng.fp8.state_dict()
        if self.model_parallel > 1:
            # every model shard of data-parallel replica 0 writes its slice; readers merge them
            pc = eng.pc
            writer = pc.dp_rank == 0 and pc.sp_rank == 0
            shards = eng.model.state_dict_shards() if writer else None
            path = self.ckpt.save(eng.step_count, {}, md, opt, rng, self.cfg.to_yaml(), extra,
                                  tensor_shards=shards,
                                  shard_rank=pc.pp_rank * pc.tp_world_size + pc.tp_rank,
                                  shard_world=pc.pp_world_size * pc.tp_world_size)
        else:
            path = self.ckpt.save(eng.step_count, eng.model.state_dict_reference(), md, opt, rng,
                                  self.cfg.to_yaml(), extra)
        self.telemetry.log("info", "checkpoint", f"saved {path}")
        return path

    def resume(self, path: str | None = None) -> dict:
        path = path or self.ckpt.latest()
        if path is None or not os.path.isdir(path):
            raise errors.CheckpointNotFound(f"no checkpoint at {path or self.ckpt.dir}")
        eng = self.engine
        md = self.ckpt.read_metadata(path)
        try:
            tensors = self.ckpt.load_tensors(path)
        except Exception as e:  # noqa: BLE001
            raise errors.CheckpointCorrupted(str(e)) from e
        eng.model.load_reference_state(tensors)
        eng.flat.refresh_master()
        mesh_now = {"pp": self.cfg.runtime.pipeline_parallel_size,
                    "tp": self.cfg.runtime.tensor_parallel_size,
                    "cp": self.cfg.runtime.context_parallel_size, "world": self.world}
        saved_mesh = (md.get("extra") or {}).get("mesh") or \
            {"pp": 1, "tp": 1, "cp": 1, "world": int(md.get("world_size", 1))}
        if self.model_parallel > 1 or any(saved_mesh[k] != 1 for k in ("pp", "tp", "cp")):
            # optimizer shards follow the model-parallel layout: they carry over only when the
            # mesh is unchanged; otherwise the moments restart (master weights come from the
            # loaded parameters)
            opt = self.ckpt.load_optimizer(path, eng.flat) if saved_mesh == mesh_now else None
            if saved_mesh != mesh_now:
                self.telemetry.log("warn", "checkpoint", f"mesh changed {saved_mesh} -> {mesh_now}: "
                                   "optimizer moments restart from zero")
        else:
            opt = self.ckpt.load_optimizer(path, eng.flat)
        if opt is not None:
            eng.flat.master.copy_(opt["master"].to(eng.flat.master))
            # Muon matrices are owned whole, round-robin over the ranks of THIS run
            owned = {s.name for i, s in enumerate(eng.optimizer._matrix_segs)
                     if i % self.world == self.rank}
            for k, v in opt.items():
                if k in ("master", "step_count"):
                    continue
                if k.startswith("muon."):
                    _, rest = k.split(".", 1)
                    name, key = rest.rsplit(".", 1)
                    if name in owned:
                        eng.optimizer._muon_state.setdefault(name, {})[key] = v.to(eng.flat.device)
                elif k.startswith("side."):
                    _, rest = k.split(".", 1)
                    name, key = rest.rsplit(".", 1)
                    eng.optimizer._side_state.setdefault(name, {})[key] = v.to(eng.flat.device)
                else:
                    eng.flat.buffer(k).copy_(v.to(eng.flat.device))
            eng.optimizer.step_count = int(opt["step_count"][0]) if "step_count" in opt \
                else int(md["step"])
        rng = self.ckpt.load_rng(path)
        if rng is not None:
            torch.set_rng_state(torch.frombuffer(bytearray(rng), dtype=torch.uint8))
        eng.step_count = int(md["step"])
        eng.tokens_seen = int(md.get("tokens_seen", 0))
        self.epoch = int(md.get("epoch", 0))
        extra = md.get("extra") or {}
        if extra.get("scheduler"):
            eng.scheduler.load_state_dict(extra["scheduler"])
        else:
            eng.scheduler.current_step = eng.step_count
        if eng.fp8 is not None:
            eng.fp8.invalidate()
            if extra.get("fp8"):
                eng.fp8.load_state_dict(extra["fp8"])
        self._resume_loader = extra.get("loader")
        if self._resume_loader and not self.cfg.data.synthetic.kind:
            self._open_data()
            self.loader.load_state_dict(self._resume_loader)
            self._open_data = lambda: None  # keep the restored cursor
        self.telemetry.log("info", "checkpoint", f"resumed {path} at step {eng.step_count}")
        return md
