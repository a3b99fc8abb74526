"""The fused compute + collective kernels on ONE GPU in loopback (every peer pointer aimed at
local memory, peer flags pre-set; see ``parallel/loopback.py``), timed with CUDA events:

    python -m ceo_b200.parallel.loopback_bench --op zero_step|ag_gemm|ag_gemm_w|gemm_rs|cp_exchange

This is the command a single-GPU profiler capture of those kernels runs (a profiler replays a
launch many times; a kernel that waits for another process cannot be replayed, one whose
"peers" are local memory can).  What loopback shows: the kernel's own instruction mix, its
DRAM traffic and tensor-pipe activity, and its time when the "link" is HBM.  What it cannot
show: NVLink bytes and link-bound time - those come from the multi-GPU runs of
``parallel/comm_bench.py`` and ``bench.py``.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from ..ops import _lib
from .loopback import BIG_EPOCH, LoopbackPeers, table


def _time(fn, iters):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=["zero_step", "ag_gemm", "ag_gemm_w", "gemm_rs", "cp_exchange"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--params", type=int, default=1 << 25, help="zero_step: flat elements")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--copy-ctas", type=int, default=0,
                    help="ag_gemm*: copy CTAs (0: 8 for activations, copy-first mode for weights; "
                         "-1: every CTA copies its share first)")
    ap.add_argument("--no-reduce", action="store_true",
                    help="zero_step: skip the reduce-scatter phase (as after bucket reductions)")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    L = _lib.lib()
    W = a.world
    peers = LoopbackPeers(W)
    st = _lib.status_word(dev)
    st.zero_()
    g = torch.Generator(device="cuda").manual_seed(0)
    rec = {"op": a.op, "world": W}

    if a.op == "zero_step":
        total = a.params
        shard = total // W
        grads = [torch.randn(total, device=dev, generator=g) * 1e-2 for _ in range(W)]
        params = [torch.zeros(total, device=dev, dtype=torch.bfloat16) for _ in range(W)]
        master, m, v = (torch.zeros(shard, device=dev) for _ in range(3))
        acc, norm, clip = torch.zeros(2, device=dev), torch.zeros(1, device=dev), torch.ones(1, device=dev)
        ranges = torch.tensor([[0, shard, 0, 1]], dtype=torch.int64, device=dev)
        peers.signal(0)
        step = [0]

        def run():
            step[0] += 1
            _lib.check(L.ceo_zero_step(table(grads), table(params), peers.flags(), peers.slots(),
                                       master.data_ptr(), m.data_ptr(), v.data_ptr(),
                                       acc.data_ptr(), norm.data_ptr(), clip.data_ptr(),
                                       st.data_ptr(), ranges.data_ptr(), 1, total, total, 0, W,
                                       peers.next_epoch(), 0, 0 if a.no_reduce else 1, 1e-3, 0.9,
                                       0.95, 1e-8, 0.1,
                                       step[0], 1.0 / W, 1.0, 0, _lib.stream()), "ceo_zero_step")
        ms = _time(run, a.iters)
        # per launch: W fp32 gradient slices read, the rank's fp32 master / m / v read + written,
        # bf16 slice stored W times, the whole local gradient buffer zeroed
        nbytes = shard * ((0 if a.no_reduce else 4 * W) + 24 + 2 * W) + total * 4
        rec.update(ms=ms, flat_elements=total, bytes=nbytes, tb_per_s=nbytes / ms / 1e9)
    elif a.op in ("ag_gemm", "ag_gemm_w"):
        M, K, N = a.tokens, a.d_model, a.n
        if a.op == "ag_gemm":     # operand 1: activations gathered over M
            bufs = [torch.randn(M, K, device=dev, generator=g).bfloat16() for _ in range(W)]
            other = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
            blk, operand, rows = 128, 1, M
        else:                     # operand 2: weight rows gathered over N (FSDP)
            bufs = [(torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16() for _ in range(W)]
            other = torch.randn(M, K, device=dev, generator=g).bfloat16()
            blk, operand, rows = math.gcd(N // W, 64), 2, N
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(rows // blk, dtype=torch.int32, device=dev)
        calls = [0]

        def run():
            calls[0] += 1
            _lib.check(L.ceo_ag_gemm_bf16(table(bufs), operand, other.data_ptr(), out.data_ptr(),
                                          M, N, K, K, N, 0, 0, 0, 1.0, None, 0, flags.data_ptr(),
                                          calls[0], 0, W, a.copy_ctas or (8 if operand == 1 else -1),
                                          blk if operand == 2 else 0, None, 0,
                                          st.data_ptr(), _lib.stream()), "ceo_ag_gemm_bf16")
        ms = _time(run, a.iters)
        rec.update(ms=ms, M=M, N=N, K=K, tflops=2.0 * M * N * K / ms / 1e9,
                   gathered_bytes=(W - 1) * (rows // W) * K * 2)
    elif a.op == "gemm_rs":
        M, N, K = a.tokens, a.d_model, a.n // 4
        rows = M // W
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
        stage = [torch.zeros(W, rows, N, dtype=torch.bfloat16, device=dev) for _ in range(W)]
        cnt = [torch.zeros(W, rows // 128, dtype=torch.int32, device=dev) for _ in range(W)]
        cnt[0][1:] = BIG_EPOCH            # the pretend peers' partial tiles "have arrived"
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
        tgt = [0]

        def run():
            tgt[0] += 4 * ((N + 255) // 256)
            _lib.check(L.ceo_gemm_rs_bf16(x.data_ptr(), w.data_ptr(), M, N, K, K, K, 0, 0, 1.0,
                                          table(stage), table(cnt), tgt[0], out.data_ptr(), None,
                                          N, 0, W, 16, st.data_ptr(), _lib.stream()),
                       "ceo_gemm_rs_bf16")
        ms = _time(run, a.iters)
        rec.update(ms=ms, M=M, N=N, K=K, tflops=2.0 * M * N * K / ms / 1e9,
                   sent_bytes=(W - 1) * rows * N * 2)
    else:
        n = 2 * 64 * 128 * 128            # (P, R) of 64 heads, d = 128
        src = torch.randn(n, device=dev, generator=g)
        gather = [torch.zeros(W * n, device=dev) for _ in range(W)]
        done = torch.zeros(1, dtype=torch.int32, device=dev)
        peers.signal(0)

        def run():
            _lib.check(L.ceo_cp_exchange(src.data_ptr(), table(gather), peers.flags(), n, 0, W,
                                         peers.next_epoch(), done.data_ptr(), st.data_ptr(),
                                         _lib.stream()), "ceo_cp_exchange")
        ms = _time(run, a.iters)
        rec.update(ms=ms, floats=n, stored_bytes=W * n * 4, gb_per_s=W * n * 4 / ms / 1e6)
    torch.cuda.synchronize()
    rec["wait_status"] = int(st.item())
    print(json.dumps(rec))
    return 0 if rec["wait_status"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
