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
    # GEMM epilogue staging at tile edges (bf16 store path), the reduce-scatter reduction and
    # the fused optimizer step in loopback (peer pointers aimed at local memory)
    from ceo_b200.ops.matmul import gemm
    from ceo_b200.parallel.loopback import LoopbackPeers, table
    a = torch.randn(200, 136, device=dev).bfloat16()
    b = torch.randn(328, 136, device=dev).bfloat16()
    r = torch.randn(200, 328, device=dev).bfloat16()
    c = gemm(a, b, residual=r)
    assert (c.float() - (a.float() @ b.float().t() + r.float())).abs().max() < 0.5
    L = _lib.lib()
    st = _lib.status_word(torch.device("cuda", 0))
    M, N, Kd = 512, 328, 64
    x = torch.randn(M, Kd, device=dev).bfloat16()
    w = torch.randn(N, Kd, device=dev).bfloat16()
    stage = [torch.zeros(2, M // 2, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    cnt = [torch.zeros(2, M // 2 // 128, dtype=torch.int32, device=dev) for _ in range(2)]
    target = 4 * ((N + 255) // 256)
    cnt[0][1] = target
    o = torch.empty(M // 2, N, dtype=torch.bfloat16, device=dev)
    _lib.check(L.ceo_gemm_rs_bf16(x.data_ptr(), w.data_ptr(), M, N, Kd, Kd, Kd, 0, 0, 1.0,
                                  table(stage), table(cnt), target, o.data_ptr(), None, N, 0, 2, 4,
                                  st.data_ptr(), _lib.stream()), "ceo_gemm_rs_bf16")
    assert (o.float() - (x.float() @ w.float().t())[:M // 2]).abs().max() < 0.5
    peers = LoopbackPeers(2)
    peers.signal(0)
    total = 4096
    gr = [torch.randn(total, device=dev) * 0.01 for _ in range(2)]
    pr = [torch.zeros(total, device=dev).bfloat16() for _ in range(2)]
    master, m1, v1 = (torch.zeros(1536, device=dev) for _ in range(3))
    rng = torch.tensor([[0, 1024, 0, 1], [2048, 512, 1024, 0]], dtype=torch.int64, device=dev)
    acc, nrm, clp = torch.zeros(2, device=dev), torch.zeros(1, device=dev), torch.ones(1, device=dev)
    _lib.check(L.ceo_zero_step(table(gr), table(pr), peers.flags(), peers.slots(), master.data_ptr(),
                               m1.data_ptr(), v1.data_ptr(), acc.data_ptr(), nrm.data_ptr(),
                               clp.data_ptr(), st.data_ptr(), rng.data_ptr(), 2, total, 2048, 0, 2,
                               peers.next_epoch(), 0, 1, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 0.5, 1.0, 0,
                               _lib.stream()), "ceo_zero_step")
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and float(master.abs().sum()) > 0
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
