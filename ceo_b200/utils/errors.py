"""Error vocabulary and finite checks (reference: src/util/error.zig:4-138)."""
from __future__ import annotations

import math


class TrainingError(RuntimeError):
    """Base of the framework's errors (the reference's ``TrainingError`` set, error.zig:4-54)."""


class ConfigInvalid(TrainingError): pass          # noqa: E701
class CheckpointCorrupted(TrainingError): pass    # noqa: E701
class CheckpointNotFound(TrainingError): pass     # noqa: E701
class DataExhausted(TrainingError): pass          # noqa: E701
class NaNDetected(TrainingError): pass            # noqa: E701
class InfDetected(TrainingError): pass            # noqa: E701
class GradientOverflow(TrainingError): pass       # noqa: E701
class LossOverflow(TrainingError): pass           # noqa: E701
class CommunicationError(TrainingError): pass     # noqa: E701
class RankFailure(CommunicationError): pass       # noqa: E701
class KernelWaitTimeout(TrainingError): pass      # noqa: E701
class OutOfMemory(TrainingError): pass            # noqa: E701
class UnsupportedDevice(TrainingError): pass      # noqa: E701
class NoGpuAvailable(TrainingError): pass         # noqa: E701
class InvalidWorldSize(TrainingError): pass       # noqa: E701
class PeerAccessUnavailable(CommunicationError): pass  # noqa: E701


class ErrorContext:
    """An error with the operation, step and rank it happened at (error.zig:90-116)."""

    def __init__(self, error: BaseException, operation: str, step: int | None = None,
                 rank: int | None = None):
        self.error, self.operation, self.step, self.rank = error, operation, step, rank

    def __str__(self):
        where = f" at step {self.step}" if self.step is not None else ""
        who = f" on rank {self.rank}" if self.rank is not None else ""
        return f"{type(self.error).__name__} during {self.operation}{where}{who}: {self.error}"


def check_finite(value: float, what: str = "value") -> float:
    """Raises NaNDetected / InfDetected (error.zig:119-129)."""
    v = float(value)
    if math.isnan(v):
        raise NaNDetected(f"{what} is NaN")
    if math.isinf(v):
        raise InfDetected(f"{what} is infinite")
    return v


def check_finite_slice(values, what: str = "values") -> None:
    for i, v in enumerate(values):
        check_finite(v, f"{what}[{i}]")
