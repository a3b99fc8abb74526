"""Data types and software codecs (reference: src/tensor/dtype.zig:3-621).

``DType`` with ``bit_size / is_quantized / accumulation_dtype / min / max`` (dtype.zig:3-83),
``ScaleFactor`` (16-deep amax history, delayed scaling: 85-128), ``BlockScale`` (130-163), and
bit-exact host codecs for FP8 E4M3 (165-261), FP8 E5M2 (263-363), BF16 with round-to-nearest
-even (365-390), FP16 (392-489) and FP4 e2m1 packed two per byte (505-553), plus
``cast_slice`` between any two of them (555-621).  The codecs are vectorised with NumPy and
serve as the oracle for ``csrc/init.cu``'s cast / FP8 kernels.
"""
from __future__ import annotations

from enum import IntEnum

import numpy as np


class DType(IntEnum):
    fp32 = 0
    fp16 = 1
    bf16 = 2
    fp8_e4m3 = 3
    fp8_e5m2 = 4
    fp4 = 5
    int8 = 6
    int32 = 7
    int64 = 8
    bool_ = 9

    def bit_size(self) -> int:
        return {0: 32, 1: 16, 2: 16, 3: 8, 4: 8, 5: 4, 6: 8, 7: 32, 8: 64, 9: 8}[int(self)]

    def is_quantized(self) -> bool:
        return self in (DType.fp8_e4m3, DType.fp8_e5m2, DType.fp4, DType.int8)

    def is_float(self) -> bool:
        return int(self) <= 5

    def accumulation_dtype(self) -> "DType":
        if self.is_float():
            return DType.fp32
        return DType.int64 if self == DType.int64 else DType.int32

    def max(self) -> float:
        return {0: 3.4028234663852886e38, 1: 65504.0, 2: 3.3895313892515355e38, 3: 448.0,
                4: 57344.0, 5: 6.0, 6: 127.0, 7: 2147483647.0, 8: 9.223372036854775807e18,
                9: 1.0}[int(self)]

    def min(self) -> float:
        return 0.0 if self == DType.bool_ else (-self.max() - (1 if self in (
            DType.int8, DType.int32, DType.int64) else 0))


# ---------------------------------------------------------------------------- bf16 / fp16
def f32_to_bf16_bits(x) -> np.ndarray:
    u = np.asarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return np.where(nan, (u >> 16) | 0x0040, rounded).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_fp16_bits(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def fp16_bits_to_f32(b) -> np.ndarray:
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


# ------------------------------------------------------------------------ generic minifloat
def _minifloat_values(exp_bits: int, man_bits: int, bias: int, ieee_inf: bool, nan_all_ones: bool):
    """Value of every non-negative code of a sign-less minifloat."""
    n = 1 << (exp_bits + man_bits)
    vals = np.empty(n, dtype=np.float64)
    for c in range(n):
        e, m = c >> man_bits, c & ((1 << man_bits) - 1)
        if e == 0:
            vals[c] = m * 2.0 ** (1 - bias - man_bits)
        else:
            vals[c] = (1 + m / (1 << man_bits)) * 2.0 ** (e - bias)
        if ieee_inf and e == (1 << exp_bits) - 1:
            vals[c] = np.inf if m == 0 else np.nan
        if nan_all_ones and c == n - 1:
            vals[c] = np.nan
    return vals


class _MiniFloat:
    def __init__(self, exp_bits, man_bits, bias, ieee_inf, nan_all_ones, max_finite):
        self.bits = 1 + exp_bits + man_bits
        self.vals = _minifloat_values(exp_bits, man_bits, bias, ieee_inf, nan_all_ones)
        finite = np.isfinite(self.vals)
        self.codes = np.nonzero(finite)[0]
        self.fvals = self.vals[finite]
        self.max_finite = max_finite
        self.sign_bit = 1 << (self.bits - 1)
        self.nan_code = int(np.nonzero(np.isnan(self.vals))[0][0]) if np.isnan(self.vals).any() \
            else None
        self.inf_code = int(np.nonzero(np.isinf(self.vals))[0][0]) if np.isinf(self.vals).any() \
            else None

    def encode(self, x, saturate: bool = True) -> np.ndarray:
        x = np.asarray(x, dtype=np.float32).astype(np.float64)
        sign = np.signbit(x)
        a = np.abs(x)
        hi = np.searchsorted(self.fvals, a, side="left").clip(0, len(self.fvals) - 1)
        lo = (hi - 1).clip(0)
        dlo, dhi = np.abs(a - self.fvals[lo]), np.abs(self.fvals[hi] - a)
        pick_lo = (dlo < dhi) | ((dlo == dhi) & (self.codes[lo] % 2 == 0))  # ties to even
        code = np.where(pick_lo, self.codes[lo], self.codes[hi])
        over = a > self.max_finite
        if saturate or self.inf_code is None:
            code = np.where(over & np.isfinite(a), self.codes[-1], code)
            code = np.where(np.isinf(a), self.codes[-1] if self.inf_code is None or saturate
                            else self.inf_code, code)
        else:
            code = np.where(over, self.inf_code, code)
        if self.nan_code is not None:
            code = np.where(np.isnan(a), self.nan_code, code)
        else:
            code = np.where(np.isnan(a), 0, code)
        return (code | np.where(sign, self.sign_bit, 0)).astype(np.uint8)

    def decode(self, c) -> np.ndarray:
        c = np.asarray(c, dtype=np.uint8).astype(np.int64)
        mag = self.vals[c & (self.sign_bit - 1)]
        return np.where(c & self.sign_bit, -mag, mag).astype(np.float32)


FP8_E4M3 = _MiniFloat(4, 3, 7, ieee_inf=False, nan_all_ones=True, max_finite=448.0)
FP8_E5M2 = _MiniFloat(5, 2, 15, ieee_inf=True, nan_all_ones=False, max_finite=57344.0)
FP4_E2M1 = _MiniFloat(2, 1, 1, ieee_inf=False, nan_all_ones=False, max_finite=6.0)


def fp4_pack(x) -> np.ndarray:
    """Two e2m1 codes per byte, low nibble first (dtype.zig:505-553)."""
    c = FP4_E2M1.encode(x) & 0xF
    if c.size % 2:
        c = np.concatenate([c, np.zeros(1, np.uint8)])
    return (c[0::2] | (c[1::2] << 4)).astype(np.uint8)


def fp4_unpack(b, n: int) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    c = np.empty(b.size * 2, np.uint8)
    c[0::2], c[1::2] = b & 0xF, b >> 4
    return FP4_E2M1.decode(c[:n])


def encode(x, dtype: DType) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    if dtype == DType.fp32:
        return x.copy()
    if dtype == DType.fp16:
        return f32_to_fp16_bits(x)
    if dtype == DType.bf16:
        return f32_to_bf16_bits(x)
    if dtype == DType.fp8_e4m3:
        return FP8_E4M3.encode(x)
    if dtype == DType.fp8_e5m2:
        return FP8_E5M2.encode(x)
    if dtype == DType.fp4:
        return fp4_pack(x)
    if dtype == DType.int8:
        return np.clip(np.rint(x), -128, 127).astype(np.int8)
    if dtype == DType.int32:
        return np.clip(np.rint(x.astype(np.float64)), -2**31, 2**31 - 1).astype(np.int32)
    if dtype == DType.int64:
        return np.rint(x.astype(np.float64)).astype(np.int64)
    return (x != 0).astype(np.uint8)


def decode(raw, dtype: DType, n: int | None = None) -> np.ndarray:
    if dtype == DType.fp32:
        return np.asarray(raw, dtype=np.float32)
    if dtype == DType.fp16:
        return fp16_bits_to_f32(raw)
    if dtype == DType.bf16:
        return bf16_bits_to_f32(raw)
    if dtype == DType.fp8_e4m3:
        return FP8_E4M3.decode(raw)
    if dtype == DType.fp8_e5m2:
        return FP8_E5M2.decode(raw)
    if dtype == DType.fp4:
        return fp4_unpack(raw, n if n is not None else 2 * np.asarray(raw).size)
    return np.asarray(raw).astype(np.float32)


def cast_slice(raw, src: DType, dst: DType, n: int | None = None) -> np.ndarray:
    """Any-to-any cast through fp32 (dtype.zig:555-621)."""
    return encode(decode(raw, src, n), dst)


class ScaleFactor:
    """Delayed scaling for FP8 tensors: the scale maps the largest magnitude of the last
    ``history`` steps onto the format's maximum (dtype.zig:85-128)."""

    def __init__(self, dtype: DType = DType.fp8_e4m3, history: int = 16, margin: int = 0):
        self.dtype, self.margin = dtype, margin
        self.amax_history = [0.0] * history
        self.cursor = 0
        self.scale = 1.0

    def update(self, amax: float) -> float:
        self.amax_history[self.cursor % len(self.amax_history)] = float(amax)
        self.cursor += 1
        m = max(self.amax_history)
        self.scale = self.dtype.max() / (m * 2.0 ** self.margin) if m > 0 and np.isfinite(m) \
            else 1.0
        return self.scale

    def inverse(self) -> float:
        return 1.0 / self.scale


class BlockScale:
    """One scale per block of ``block`` consecutive elements (dtype.zig:130-163)."""

    def __init__(self, block: int = 32, dtype: DType = DType.fp8_e4m3):
        self.block, self.dtype = block, dtype

    def quantize(self, x):
        x = np.asarray(x, dtype=np.float32)
        pad = (-x.size) % self.block
        xp = np.concatenate([x.ravel(), np.zeros(pad, np.float32)]).reshape(-1, self.block)
        amax = np.abs(xp).max(axis=1)
        scales = np.where(amax > 0, self.dtype.max() / amax, 1.0).astype(np.float32)
        q = encode((xp * scales[:, None]).ravel(), self.dtype)
        return q, scales

    def dequantize(self, q, scales, n: int):
        v = decode(q, self.dtype, scales.size * self.block).reshape(-1, self.block)
        return (v / scales[:, None]).ravel()[:n]
