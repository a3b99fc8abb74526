"""Failure detection and recovery on the host.

The reference has error enums, ``checkFinite`` and an unused ``ncclCommAbort`` binding but no
heartbeat, watchdog or recovery path (src/runtime/nccl.zig:84, src/util/error.zig:119-129,
src/telemetry/main.zig:113-177; its cloud launcher sets ``retries=0``).  This module adds:

* ``Heartbeat``: every rank publishes a monotonically increasing beat in the rendezvous
  store; ``dead_ranks`` lists ranks whose beat has not moved for ``timeout`` seconds.  Ranks
  consult it between steps, before launching kernels that wait on peers.
* ``KernelWatch``: reads the device status word that kernels with bounded waits set when a
  wait ran out (the kernel itself returns normally, the context stays usable) and turns it
  into ``KernelWaitTimeout`` naming the kernel phase and peer.
* ``StepGuard``: wraps a training step; on a dead peer, a kernel wait time-out, a collective
  error or a non-finite loss it raises a typed error so the driver loop (``run_with_recovery``)
  can tear the process group down, re-rendezvous with the survivors and resume from the
  newest checkpoint.
* ``FaultInjector``: host-side injection for tests (raise in a step, skip a heartbeat, drop a
  store key, corrupt a checkpoint byte).  Nothing here faults, traps or hangs a device.
"""
from __future__ import annotations

import math
import os
import threading
import time

from ..utils import errors


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval: float = 0.5, timeout: float = 5.0,
                 prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._beat = 0
        self._seen = {r: (None, time.time()) for r in range(world)}
        self._stop = threading.Event()
        self._paused = False
        self._thread = None

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self):
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))

    def start(self):
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                if not self._paused:
                    try:
                        self.beat()
                    except Exception:  # noqa: BLE001  store gone: the job is ending
                        return
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def pause(self, paused: bool = True):
        """Test hook: stop publishing without stopping the process."""
        self._paused = paused

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def _read(self, r: int):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return self.store.get(self._key(r)).decode()
        except Exception:  # noqa: BLE001
            return None

    def dead_ranks(self) -> list[int]:
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            val = self._read(r)
            last, since = self._seen[r]
            if val is not None and val != last:
                self._seen[r] = (val, now)
            elif now - since > self.timeout:
                dead.append(r)
        return dead

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise errors.RankFailure(f"no heartbeat from rank(s) {dead} for {self.timeout:.1f}s")


WAIT_CODES = {1: "gemm: TMA producer waiting for a free stage", 2: "gemm: MMA waiting for data",
              3: "gemm: MMA waiting for a free accumulator", 4: "gemm: epilogue waiting for MMA",
              5: "all-gather gemm: TMA producer waiting for a peer's row block to be copied in",
              6: "gemm reduce-scatter: reduction waiting for a peer's partial tiles",
              7: "all-gather gemm: copy CTA waiting for a bulk copy from a peer",
              0x4546: "efla: a tile or pipeline wait ran out"}


def describe_status(code: int) -> str:
    """What a non-zero device status word means (the code the first bounded wait that ran out
    wrote: csrc/gemm_tcgen05.cu ST_*, csrc/efla.cu EFLA_WAIT_STATUS, csrc/comm.cu
    100 + 10 * barrier slot + missing rank)."""
    if code in WAIT_CODES:
        return WAIT_CODES[code]
    if 100 <= code < 200:
        slot, peer = (code - 100) // 10, (code - 100) % 10
        return f"peer barrier {slot}: no signal from rank {peer}"
    return f"status {code}"


class KernelWatch:
    def __init__(self, read_status=None, reset_status=None):
        if read_status is None:
            from ..ops import _lib
            read_status = _lib.read_status

            def reset_status():
                import torch
                _lib.status_word(torch.device("cuda", torch.cuda.current_device())).zero_()
        self._read, self._reset = read_status, reset_status

    def check(self):
        code = int(self._read())
        if code != 0:
            if self._reset is not None:
                self._reset()
            raise errors.KernelWaitTimeout(describe_status(code))


class StepGuard:
    def __init__(self, heartbeat: Heartbeat | None = None, kernel_watch: KernelWatch | None = None,
                 check_every: int = 1):
        self.hb, self.kw, self.every = heartbeat, kernel_watch, max(1, check_every)
        self.steps = 0

    def before_step(self):
        if self.hb is not None:
            self.hb.check()

    def after_step(self, loss=None):
        self.steps += 1
        if loss is not None and self.steps % self.every == 0:
            v = float(loss)
            if math.isnan(v):
                raise errors.NaNDetected(f"loss is NaN at guarded step {self.steps}")
            if math.isinf(v):
                raise errors.InfDetected(f"loss is infinite at guarded step {self.steps}")
        if self.kw is not None and self.steps % self.every == 0:
            self.kw.check()

    def run(self, fn, *a, **kw):
        self.before_step()
        try:
            out = fn(*a, **kw)
        except RuntimeError as e:  # a collective that timed out or was aborted
            msg = str(e)
            if any(s in msg for s in ("NCCL", "Gloo", "timed out", "Connection", "connection")):
                raise errors.CommunicationError(msg) from e
            raise
        loss = out[0] if isinstance(out, tuple) else None
        self.after_step(loss)
        return out


class FaultInjector:
    """Host-side faults for tests."""

    def __init__(self):
        self.fail_at_step = None
        self.exc = RuntimeError("injected failure")

    def maybe_raise(self, step: int):
        if self.fail_at_step is not None and step == self.fail_at_step:
            self.fail_at_step = None
            raise self.exc

    @staticmethod
    def corrupt_file(path: str, offset_from_end: int = 1):
        with open(path, "r+b") as f:
            f.seek(-offset_from_end, os.SEEK_END)
            b = f.read(1)
            f.seek(-offset_from_end, os.SEEK_END)
            f.write(bytes([b[0] ^ 0xFF]))

    @staticmethod
    def drop_key(store, key: str):
        if hasattr(store, "delete_key"):
            store.delete_key(key)


def run_with_recovery(make_trainer, total_steps: int, max_restarts: int = 2, on_restart=None):
    """Drives ``trainer.run`` and, on a recoverable error, rebuilds the trainer (which
    re-rendezvouses and resumes from the newest valid checkpoint) up to ``max_restarts`` times.
    ``make_trainer(attempt)`` returns an object with ``run(max_steps)``, ``resume()``,
    ``engine.step_count`` and ``ckpt.latest()``."""
    attempt = 0
    while True:
        tr = make_trainer(attempt)
        if tr.ckpt.latest() is not None:
            try:
                tr.resume()
            except errors.CheckpointCorrupted:
                # fall back to the previous checkpoint
                steps = tr.ckpt.list_checkpoints()
                if len(steps) < 2:
                    raise
                tr.resume(tr.ckpt.path_for(steps[-2]))
        try:
            remaining = total_steps - tr.engine.step_count
            if remaining > 0:
                tr.run(max_steps=remaining)
            return tr
        except (errors.RankFailure, errors.CommunicationError, errors.KernelWaitTimeout,
                errors.NaNDetected, errors.InfDetected, RuntimeError) as e:
            attempt += 1
            if attempt > max_restarts:
                raise
            if on_restart is not None:
                on_restart(attempt, e)
