"""Runs a set of ops on the bounds-checked build of the kernel library (the parent test sets
CEO_B200_BOUNDS_CHECK=1) and prints what the checker recorded."""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ceo_b200.ops import _lib, nn as K, tensor_ops as TO  # noqa: E402


def main():
    assert _lib.BOUNDS_CHECK and _lib.LIB_PATH.name == "libceo_b200_chk.so"
    dev = "cuda"
    torch.manual_seed(0)
    out = {}
    assert _lib.bounds_status() == (0, 0, 0, 0)
    # tile-edge shapes through the instrumented kernels, each against its oracle
    table = torch.randn(1000, 264, device=dev).bfloat16()
    ids = torch.randint(0, 1000, (3, 77), device=dev)
    assert torch.equal(K.embedding(ids, table), table[ids])
    src = torch.randn(333, 24, device=dev)
    idx = torch.randint(0, 333, (500,), device=dev)
    assert torch.equal(TO.gather_rows(src, idx), src[idx])
    dst = torch.zeros(333, 24, device=dev)
    perm = torch.randperm(333, device=dev)
    TO.scatter_rows(dst, perm, src)
    assert torch.equal(dst[perm], src)
    acc = torch.zeros(50, 24, device=dev)
    i2 = torch.randint(0, 50, (333,), device=dev)
    TO.scatter_add_rows(acc, i2, src)
    assert torch.allclose(acc, torch.zeros(50, 24, device=dev).index_add_(0, i2, src), atol=1e-4)
    x = torch.randn(130, 70, device=dev).bfloat16()
    assert torch.equal(TO.transpose2d(x), x.t().contiguous())
    gu = torch.randn(37, 2 * 264, device=dev).bfloat16()
    g, u = gu[:, :264].float(), gu[:, 264:].float()
    assert (K.swiglu(gu).float() - g * torch.sigmoid(g) * u).abs().max() < 0.05
    out["clean"] = _lib.bounds_status()
    # the recorder itself: 5 indices past the end of a 100-element buffer, redirected to 0
    buf = torch.ones(101, device=dev)
    buf[100] = 0
    rc = _lib.lib().ceo_bounds_selftest(buf.data_ptr(), 100, 5, _lib.stream())
    assert rc == 0
    out["selftest"] = _lib.bounds_status()
    out["after_reset"] = _lib.bounds_status()
    out["sum"] = float(buf[100])
    print("BOUNDS " + json.dumps(out))


if __name__ == "__main__":
    main()
