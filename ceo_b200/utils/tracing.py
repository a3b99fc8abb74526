"""In-process tracing: NVTX ranges around the phases of a training step (visible in any
CUDA timeline tool) and a per-kernel time table of one call through ``torch.profiler``.

The reference has no in-process tracing at all: ``enable-profiling`` links CUPTI but no
source tests the macro (build.zig:19,53-56), ``efla-train profile`` only prints hints
(src/main.zig:476-483) and scripts/profile.sh wraps the external profilers.

Ranges cost one branch when tracing is off (the default; ``CEO_TRACE=1`` or
``set_enabled(True)`` turns it on).  The profiler table is a diagnostic: numbers taken under
a profiler are never benchmark values.
"""
from __future__ import annotations

import contextlib
import os

import torch

_enabled = os.environ.get("CEO_TRACE", "0") not in ("", "0", "false", "False")


def set_enabled(on: bool) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def trace_range(name: str):
    """NVTX range ``name`` around the block (no-op when tracing is off or without CUDA)."""
    if _enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def kernel_table(fn, warmup: int = 1) -> dict:
    """Runs ``fn()`` under the profiler once (after ``warmup`` plain calls) and returns
    ``{"busy_ms", "span_ms", "kernels": [(name, launches, ms), ...]}`` sorted by time."""
    from torch.profiler import ProfilerActivity, profile
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        fn()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    tot: dict[str, list] = {}
    for e in ev:
        t = tot.setdefault(e.name.split("(")[0], [0, 0.0])
        t[0] += 1
        t[1] += getattr(e, "device_time", None) or e.cuda_time
    spans = sorted((e.time_range.start, e.time_range.end) for e in ev)
    span = (spans[-1][1] - spans[0][0]) if spans else 0.0
    rows = sorted(((k, v[0], v[1] / 1e3) for k, v in tot.items()), key=lambda r: -r[2])
    return {"busy_ms": sum(r[2] for r in rows), "span_ms": span / 1e3, "kernels": rows}


def format_table(table: dict, top: int = 30) -> str:
    busy = table["busy_ms"] or 1.0
    lines = [f"kernels busy {table['busy_ms']:.2f} ms over a span of {table['span_ms']:.2f} ms",
             f"{'ms':>10} {'share':>7} {'launches':>9}  kernel"]
    for name, n, ms in table["kernels"][:top]:
        lines.append(f"{ms:10.3f} {100 * ms / busy:6.1f}% {n:9d}  {name[:90]}")
    return "\n".join(lines)
