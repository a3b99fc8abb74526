"""Builds the sm_100a kernel library in-tree: ``ceo_b200/lib/libceo_b200.so``.

Each ``csrc/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` into an object file
(in parallel, skipped when the object is newer than every source it depends on)
and the objects are linked into one shared library with a plain C ABI
(``csrc/include/ceo_kernels.h``).  No GPU is needed to build.

Counterpart of the reference's kernel build step (build.zig:144-186,
scripts/build_kernels.sh:45-77), which lists sources that do not exist and
targets plain ``sm_100``.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "lib" / "obj"
LIB = ROOT / "lib" / "libceo_b200.so"
# debug variant with checked indexing (csrc/common/check.cuh); loaded when CEO_B200_BOUNDS_CHECK=1
OBJ_CHK = ROOT / "lib" / "obj_chk"
LIB_CHK = ROOT / "lib" / "libceo_b200_chk.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
    f"-I{CSRC}",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the kernel library cannot be built")
    return cand


def _deps_mtime() -> float:
    hdrs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _compile(src: Path, hdr_mtime: float, verbose: bool, extra: list[str],
             objdir: Path = OBJ) -> tuple[Path, str]:
    obj = objdir / (src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime) and not extra:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(verbose: bool = False, force: bool = False, extra: list[str] | None = None,
          bounds_check: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library
    (``bounds_check``: the debug variant with checked indexing, a separate file)."""
    extra = list(extra or [])
    objdir, lib = (OBJ_CHK, LIB_CHK) if bounds_check else (OBJ, LIB)
    if bounds_check:
        extra.append("-DCEO_BOUNDS_CHECK")
        force = True
    objdir.mkdir(parents=True, exist_ok=True)
    if force:
        for o in objdir.glob("*.o"):
            o.unlink()
    hdr_mtime = _deps_mtime()
    srcs = sources()
    objs: list[Path] = []
    logs: list[str] = []
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        for obj, log in ex.map(lambda s: _compile(s, hdr_mtime, verbose, extra, objdir), srcs):
            objs.append(obj)
            if log:
                logs.append(log)
    newest = max(o.stat().st_mtime for o in objs)
    if force or not lib.exists() or lib.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print("\n".join(logs))
    return lib


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="-f" in sys.argv,
              bounds_check="--bounds-check" in sys.argv)
    print(p)
