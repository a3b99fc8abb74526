"""Telemetry: text log, JSONL step records, Prometheus text exposition, rolling stats,
health checks.

File names, record fields and line formats follow the reference's Telemetry
(src/telemetry/main.zig:20-294): rank 0 appends to ``log_file`` and ``{log_file}.jsonl``;
``log_step`` writes ``{step,tokens,lr,grad_norm,timestamp}`` (main.zig:69-86); ``log_metrics``
writes ``[ts] step= loss= lr= tokens= throughput=`` (main.zig:89-110).  The reference's
Prometheus export prints three gauges with literal zeros and has no server
(main.zig:120-134); here the gauges carry the last values and an optional HTTP endpoint
serves them on ``prometheus_port``.  ``throughput`` is device-timed tokens per second, not
the reference's tokens-per-step ratio (src/runtime/trainer.zig:313-314).
"""
from __future__ import annotations

import json
import math
import sys
import threading
import time
from collections import deque

LEVELS = {"debug": 0, "info": 1, "warn": 2, "err": 3}


def _ts() -> int:
    return int(time.time())


def log(level: str, scope: str, msg: str, min_level: str = "info", stream=None) -> None:
    """``[ts] [LEVEL] scope: msg`` on stderr (main.zig:180-204)."""
    if LEVELS[level] >= LEVELS[min_level]:
        print(f"[{_ts()}] [{level.upper()}] {scope}: {msg}", file=stream or sys.stderr)


class TrainingStats:
    """Rolling loss mean and tokens/s over a window (main.zig:237-294)."""

    def __init__(self, window: int = 100):
        self.losses = deque(maxlen=window)
        self.tokens = 0
        self.t0 = time.time()
        self.samples = deque(maxlen=window)

    def update(self, loss: float, tokens: int, seconds: float | None = None):
        self.losses.append(loss)
        self.tokens += tokens
        if seconds is not None and seconds > 0:
            self.samples.append((tokens, seconds))

    def avg_loss(self) -> float:
        return sum(self.losses) / len(self.losses) if self.losses else 0.0

    def tokens_per_sec(self) -> float:
        if self.samples:
            return sum(t for t, _ in self.samples) / sum(s for _, s in self.samples)
        dt = time.time() - self.t0
        return self.tokens / dt if dt > 0 else 0.0


class MemoryStats:
    """allocated / reserved / peak bytes (main.zig:207-234), from the CUDA caching allocator."""

    def __init__(self):
        self.allocated = self.reserved = self.peak = self.free = self.total = 0

    def update(self):
        try:
            import torch
            if torch.cuda.is_available():
                self.allocated = torch.cuda.memory_allocated()
                self.reserved = torch.cuda.memory_reserved()
                self.peak = torch.cuda.max_memory_allocated()
                self.free, self.total = torch.cuda.mem_get_info()
        except Exception:  # noqa: BLE001
            pass
        return self


class HealthStatus:
    """gpu / memory / nan_inf / temperature flags (main.zig:113-118)."""

    def __init__(self, gpu_ok=True, memory_ok=True, nan_inf=False, temperature_ok=True):
        self.gpu_ok, self.memory_ok = gpu_ok, memory_ok
        self.nan_inf, self.temperature_ok = nan_inf, temperature_ok

    def healthy(self) -> bool:
        return self.gpu_ok and self.memory_ok and not self.nan_inf and self.temperature_ok


def check_nan_inf(values) -> bool:
    """True if any value is NaN or infinite (main.zig:170-177)."""
    return any((not math.isfinite(float(v))) for v in values)


class Telemetry:
    def __init__(self, cfg=None, rank: int = 0, log_file: str | None = None,
                 log_level: str = "info", enable_prometheus: bool = False,
                 prometheus_port: int = 9090):
        if cfg is not None:
            log_file = cfg.log_file if log_file is None else log_file
            log_level, enable_prometheus = cfg.log_level, cfg.enable_prometheus
            prometheus_port = cfg.prometheus_port
        self.rank, self.level = rank, log_level
        self.text = self.jsonl = None
        if rank == 0 and log_file:
            self.text = open(log_file, "a", buffering=1)
            self.jsonl = open(log_file + ".jsonl", "a", buffering=1)
        self.gauges = {"efla_training_loss": 0.0, "efla_tokens_per_second": 0.0,
                       "efla_gpu_memory_bytes": 0.0, "efla_learning_rate": 0.0,
                       "efla_grad_norm": 0.0, "efla_step": 0.0, "efla_mfu": 0.0}
        self.stats = TrainingStats()
        self.memory = MemoryStats()
        self._server = None
        if rank == 0 and enable_prometheus:
            self.start_prometheus(prometheus_port)

    def log(self, level: str, scope: str, msg: str):
        if self.rank == 0:
            log(level, scope, msg, self.level)
            if self.text and LEVELS[level] >= LEVELS[self.level]:
                self.text.write(f"[{_ts()}] [{level.upper()}] {scope}: {msg}\n")

    def log_step(self, step: int, tokens: int, lr: float, grad_norm: float):
        self.gauges.update(efla_learning_rate=lr, efla_grad_norm=grad_norm, efla_step=step)
        if self.jsonl:
            self.jsonl.write(json.dumps({"step": step, "tokens": tokens, "lr": lr,
                                         "grad_norm": grad_norm, "timestamp": _ts()}) + "\n")

    def log_metrics(self, step: int, loss: float, lr: float, tokens: int, throughput: float,
                    mfu: float | None = None):
        self.gauges.update(efla_training_loss=loss, efla_tokens_per_second=throughput,
                           efla_gpu_memory_bytes=float(self.memory.update().allocated))
        line = (f"[{_ts()}] step={step} loss={loss:.4f} lr={lr:.6e} tokens={tokens} "
                f"throughput={throughput:.2f}")
        if mfu is not None:
            self.gauges["efla_mfu"] = mfu
            line += f" mfu={mfu:.4f}"
        if self.text:
            self.text.write(line + "\n")
        if self.rank == 0:
            print(line, file=sys.stderr)

    def log_health_check(self, status: HealthStatus):
        self.log("info" if status.healthy() else "warn", "health",
                 f"gpu={status.gpu_ok} memory={status.memory_ok} nan_inf={status.nan_inf} "
                 f"temperature={status.temperature_ok}")

    def export_prometheus(self) -> str:
        out = []
        for k, v in self.gauges.items():
            out.append(f"# TYPE {k} gauge")
            out.append(f"{k} {v}")
        return "\n".join(out) + "\n"

    def start_prometheus(self, port: int):
        from http.server import BaseHTTPRequestHandler, HTTPServer
        tel = self

        class H(BaseHTTPRequestHandler):
            def do_GET(self):  # noqa: N802
                body = tel.export_prometheus().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass
        self._server = HTTPServer(("127.0.0.1", port), H)
        threading.Thread(target=self._server.serve_forever, daemon=True).start()
        return self._server.server_address[1]

    def close(self):
        if self._server is not None:
            self._server.shutdown()
            self._server = None
        for f in (self.text, self.jsonl):
            if f:
                f.close()
        self.text = self.jsonl = None
