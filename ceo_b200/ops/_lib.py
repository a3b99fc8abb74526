"""ctypes loader for the in-tree kernel library ``ceo_b200/lib/libceo_b200.so``.

Argument types are generated from the C header (``csrc/include/ceo_kernels.h``)
so the Python shims cannot drift from the ABI: every pointer is passed as a
64-bit address, ``long long`` as 64-bit, ``cudaStream_t`` as the raw handle of
the current torch stream.

On a machine with a GPU a missing library is an error (no silent fallback to
PyTorch); without a GPU the ops run their fp32 PyTorch oracles and the library
is not needed.  Same role as the extern blocks of the reference's
src/kernels/{efla,nn,optim,prism}_kernels.zig.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
# CEO_B200_BOUNDS_CHECK=1 selects the debug build with checked indexing
# (`python -m ceo_b200.build --bounds-check`); see bounds_status().
BOUNDS_CHECK = os.environ.get("CEO_B200_BOUNDS_CHECK", "0") not in ("", "0")
LIB_PATH = _PKG / "lib" / ("libceo_b200_chk.so" if BOUNDS_CHECK else "libceo_b200.so")
HEADER_PATH = _PKG / "csrc" / "include" / "ceo_kernels.h"

_lib = None
_status = {}
_scratch = {}

# kernels launched per entry point (everything not listed launches exactly one)
_LAUNCHES = {"ceo_efla_fwd": 3, "ceo_efla_bwd": 3, "ceo_rmsnorm_bwd": 2, "ceo_layernorm_bwd": 4,
             "ceo_sumsq": 2, "ceo_reduce": 2, "ceo_muon_momentum": 2, "ceo_norm_bwd_blocks": 0,
             "ceo_sumsq_blocks": 0, "ceo_reduce_blocks": 0, "ceo_cumsum_scratch_floats": 0,
             "ceo_efla_set_tcgen05": 0, "ceo_bounds_status": 0, "ceo_fp8_quantize": 1,
             "ceo_zero_bucket_reduce": 2, "ceo_set_wait_limit": 0, "ceo_gemm_set_wait_limit": 0,
             "ceo_efla_set_wait_limit": 0, "ceo_set_deterministic": 0, "ceo_dev_malloc": 0,
             "ceo_dev_free": 0, "ceo_ipc_get_handle": 0, "ceo_ipc_open": 0, "ceo_ipc_close": 0}
launch_count = 0


class _Counted:
    """Wraps a ctypes entry point and counts the kernels it launches."""
    __slots__ = ("fn", "n")

    def __init__(self, fn, n):
        self.fn, self.n = fn, n

    def __call__(self, *a):
        global launch_count
        launch_count += self.n
        return self.fn(*a)


class _Lib:
    pass

_CTYPE = {
    "int": ctypes.c_int,
    "float": ctypes.c_float,
    "long long": ctypes.c_longlong,
    "cudaStream_t": ctypes.c_void_p,
    "size_t": ctypes.c_size_t,
}


def _parse_header(text: str) -> dict[str, list]:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    protos = {}
    for m in re.finditer(r"\bint\s+(ceo_\w+)\s*\(([^)]*)\)\s*;", text):
        name, args = m.group(1), m.group(2).strip()
        types = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    types.append(ctypes.c_void_p)
                    continue
                a = a.replace("const ", "").replace("unsigned ", "")
                base = a.rsplit(" ", 1)[0] if " " in a else a
                types.append(_CTYPE[base])
        protos[name] = types
    return protos


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    """The loaded kernel library (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ceo_b200.build` "
                "(CUDA tensors are never routed to a PyTorch fallback)")
        cdll = ctypes.CDLL(str(LIB_PATH))
        wrapped = _Lib()
        wrapped.cdll = cdll
        for name, argtypes in _parse_header(HEADER_PATH.read_text()).items():
            fn = getattr(cdll, name, None)
            if fn is None:
                raise RuntimeError(f"{name} is declared in ceo_kernels.h but not exported")
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
            setattr(wrapped, name, _Counted(fn, _LAUNCHES.get(name, 1)))
        _lib = wrapped
    return _lib


class KernelError(RuntimeError):
    pass


_NEG = {-2: "misaligned pointer or stride", -3: "tensor map for A rejected",
        -4: "tensor map for B rejected", -5: "unsupported shape or dtype"}


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: {_NEG.get(rc, 'argument error')} (code {rc})")
    raise KernelError(f"{what}: CUDA error {rc}")


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status_word(device: torch.device) -> torch.Tensor:
    """Device int32 that kernels with bounded waits set when a wait ran out."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def read_status(device: torch.device | None = None) -> int:
    """Host read (synchronises) of the wait-status word; 0 means no wait ever gave up."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    return int(status_word(device).item())


def bounds_status(reset: bool = True):
    """Checked build: ``(violations, site, index, extent)`` of the first out-of-range index the
    kernels recorded (synchronises the device).  Normal build: ``None``."""
    out = (ctypes.c_longlong * 4)()
    rc = lib().ceo_bounds_status(ctypes.addressof(out), int(reset))
    if rc == -1:
        return None
    check(rc, "ceo_bounds_status")
    return tuple(int(v) for v in out)


def scratch(device: torch.device, nfloats: int, tag: str = "f32") -> torch.Tensor:
    """A cached fp32 scratch buffer of at least `nfloats` elements (per device and tag)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1 << 16), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf
