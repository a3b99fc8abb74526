"""Builds the reference's own CUDA kernels into ``baseline/_ref/libref_kernels.so`` so they can
be timed on the same GPU as this framework's kernels (``baseline/ref_kernel_bench.py``).

The sources are compiled as shipped with the reference's flags (``-arch=sm_100 -O3
--use_fast_math``, build.zig:165-175), with one exception: ``efla.cu`` lines 130-152 hold a
dead kernel that uses an undeclared identifier and does not compile, so those lines are left
out of the copy that is built.  Nothing of the reference is committed: the copies and the
library live under the git-ignored ``baseline/_ref``.
Usage: ``python baseline/build_ref_kernels.py /path/to/reference`` (or the path in the
environment variable ``CEO_REFERENCE_DIR``).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def main(ref=None):
    ref = ref or os.environ.get("CEO_REFERENCE_DIR")
    if not ref:
        print("usage: build_ref_kernels.py <reference tree>  (or set CEO_REFERENCE_DIR)")
        return 2
    src = os.path.join(ref, "kernels", "cuda")
    if not os.path.isdir(src):
        print(f"reference kernels not found at {src}")
        return 1
    work = os.path.join(OUT, "kernels")
    shutil.rmtree(work, ignore_errors=True)
    shutil.copytree(src, work)
    lines = open(os.path.join(work, "efla.cu")).read().split("\n")
    kept = lines[:129] + lines[152:]          # drop the dead stub (1-based lines 130-152)
    open(os.path.join(work, "efla_nostub.cu"), "w").write("\n".join(kept))
    files = ["gemm.cu", "layernorm.cu", "optim.cu", "init.cu", "efla_nostub.cu"]
    cmd = ["nvcc", "-arch=sm_100", "-O3", "--use_fast_math", "-DCUDA_ARCH_SM100", "-shared",
           "-Xcompiler", "-fPIC", "-I" + os.path.join(work, "include"),
           *[os.path.join(work, f) for f in files], "-lcublas", "-o",
           os.path.join(OUT, "libref_kernels.so")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    print(r.stdout[-2000:], r.stderr[-2000:])
    return r.returncode


if __name__ == "__main__":
    sys.exit(main(*sys.argv[1:2]))
