"""Chunked EFLA forward+backward microbenchmark with context parallelism:
``python -m ceo_b200.parallel.cp_bench`` (1 GPU) or under ``torchrun --nproc-per-node N``.

B=4, H=16, d_k=d_v=128, T=65536 split over the N ranks; q/k ~ N(0,1) then L2-normalised,
v ~ N(0,1), beta = sigmoid(N(0,1)), all from a seed.  Reports the matmul TFLOP/s of the whole
job (forward + backward, the FLOP count of ``parallel.cp.efla_flops``), the fraction of the
measured bf16 GEMM peak, and the time of the inter-rank state exchange alone.  CUDA events,
max over ranks, inputs (several GB) far larger than L2.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from ..ops import efla
from ..utils.kernel_bench import peaks
from .comm import Comm, init_distributed
from .cp import CPContext, cp_delta_rule, efla_flops


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--seq-len", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    rank, world, local = init_distributed()
    torch.cuda.set_device(local)
    B, H, d, T = a.batch, a.heads, a.head_dim, a.seq_len
    Tl = T // world
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    q = torch.randn(B, Tl, H, d, device="cuda", generator=g)
    k = torch.randn(B, Tl, H, d, device="cuda", generator=g)
    q = (q / q.norm(dim=-1, keepdim=True)).bfloat16().requires_grad_()
    k = (k / k.norm(dim=-1, keepdim=True)).bfloat16().requires_grad_()
    v = torch.randn(B, Tl, H, d, device="cuda", generator=g).bfloat16().requires_grad_()
    alpha = (-torch.expm1(-torch.sigmoid(torch.randn(B, Tl, H, device="cuda", generator=g)))) \
        .requires_grad_()
    do = torch.randn(B, Tl, H, d, device="cuda", generator=g).bfloat16()
    comm = cp = None
    if world > 1:
        from .fused import FusedComm
        comm = FusedComm()
        cp = CPContext(comm, B * H, d)

    def step():
        if cp is None:
            o, _ = efla.delta_rule(q, k, v, alpha)
        else:
            o = cp_delta_rule(q, k, v, alpha, cp)
        torch.autograd.grad(o, (q, k, v, alpha), do)

    def timed(fn, iters):
        ts = []
        for _ in range(iters):
            if comm is not None:
                comm.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            ts.append(comm.max_over_ranks(ms) if comm is not None else ms)
        return statistics.median(ts)

    for _ in range(a.warmup):
        step()
    ms = timed(step, a.iters)
    ex_ms = None
    if cp is not None:
        blk = torch.randn(2, B, H, d, d, device="cuda")
        ex_ms = timed(lambda: cp.exchange(blk), a.iters)
    flops = efla_flops(B, T, H, d, True)
    _, peak, kind = peaks()
    if rank == 0:
        print(json.dumps({
            "op": "chunked EFLA fwd+bwd, context parallel", "n_gpus": world, "B": B, "H": H,
            "d": d, "T": T, "ms": round(ms, 3), "tflops_total": round(flops / ms / 1e9, 1),
            "tflops_per_gpu": round(flops / ms / 1e9 / world, 1),
            f"frac_of_{kind}_gemm_peak_per_gpu": round(flops / (ms * 1e-3) / world / peak, 4),
            "state_exchange_ms": None if ex_ms is None else round(ex_ms, 4),
            "exchange_bytes_per_rank": 2 * B * H * d * d * 4 * max(0, world - 1)}))
    if cp is not None:
        cp.close()
        comm.close()
    Comm().barrier()


if __name__ == "__main__":
    main()
