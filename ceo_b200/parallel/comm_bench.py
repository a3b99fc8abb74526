"""Fused compute+collective kernels against their NCCL compositions, with roofline fractions:
``torchrun --nproc-per-node N -m ceo_b200.parallel.comm_bench``.

For each op the target time is the slower of FLOPs / measured GEMM peak and bytes that must
cross NVLink / 770 GB/s (the measured per-direction peer-copy rate; nominal 900); the table
reports achieved / target for the fused kernel and the time of the NCCL composition.  Timed
with CUDA events after warm-up, max over ranks, an L2 flush before every timed launch.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch
import torch.distributed as dist

from ..utils.kernel_bench import peaks
from .comm import Comm, init_distributed
from .fused import FusedComm
from .tp import TPContext

NVLINK_BPS = 770e9


def timed(fn, comm, iters=8, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        comm.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(comm.max_over_ranks(e0.elapsed_time(e1)))
    return statistics.median(ts)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", choices=["", "tp", "fsdp"],
                    help="tp: the tensor-parallel rows; fsdp: the weight-gather rows")
    a = ap.parse_args(argv)
    rank, world, local = init_distributed()
    torch.cuda.set_device(local)
    fc = FusedComm()
    _, flops_peak, kind = peaks()
    M, D = a.tokens, a.d_model
    rows = M // world
    out = []

    def rec(name, fused_ms, nccl_ms, flops, link_bytes):
        target = max(flops / flops_peak, link_bytes / NVLINK_BPS) * 1e3
        r = {"op": name, "world": world, "fused_ms": round(fused_ms, 4),
             "nccl_ms": round(nccl_ms, 4), "speedup_vs_nccl": round(nccl_ms / fused_ms, 3),
             "roofline_ms": round(target, 4),
             f"frac_of_roofline_{kind}": round(target / fused_ms, 3)}
        out.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    ncol = max(3 * D // world, 256)
    ffn_loc = (a.ffn // world + 255) // 256 * 256
    tp = TPContext(fc, M, max(D, ncol, ffn_loc, 2 * ffn_loc))
    g = torch.Generator(device="cuda").manual_seed(rank)
    xs = torch.randn(rows, D, device="cuda", generator=g).bfloat16()
    from ..ops.matmul import gemm as plain_gemm
    tp_rows = a.only in ("", "tp")
    t_bar = timed(lambda: fc.device_barrier(), fc)
    if rank == 0:
        print(json.dumps({"op": "device barrier (flag kernel)", "world": world,
                          "ms": round(t_bar, 4)}), flush=True)
    for name, n_loc in (("ag_gemm qkv", ncol), ("ag_gemm gate_up", 2 * ffn_loc)) if tp_rows else ():
        w = (torch.randn(n_loc, D, device="cuda", generator=g) * 0.02).bfloat16()
        f = timed(lambda: tp.ag_gemm(xs, w), fc)          # the default choice of mode
        tp.copy_ctas = 8
        f_cc = timed(lambda: tp.ag_gemm(xs, w), fc)       # dedicated copy CTAs
        tp.copy_ctas = -1
        n = timed(lambda: tp.ag_gemm_nccl(xs, w), fc)
        xf = torch.randn(M, D, device="cuda", generator=g).bfloat16()
        loc = timed(lambda: plain_gemm(xf, w), fc)
        rec(f"{name} {M}x{n_loc}x{D}", f, n, 2.0 * M * n_loc * D,
            (world - 1) / world * M * D * 2)
        out[-1]["local_gemm_ms"] = round(loc, 4)
        out[-1]["fused_copy_ctas_ms"] = round(f_cc, 4)
        if rank == 0:
            print(json.dumps({"local_gemm_ms": round(loc, 4), "fused_copy_ctas_ms": round(f_cc, 4)}),
                  flush=True)
    for name, k_loc in (("gemm_rs out", max(D // world, 256)),
                        ("gemm_rs down", ffn_loc)) if tp_rows else ():
        x = torch.randn(M, k_loc, device="cuda", generator=g).bfloat16()
        w = (torch.randn(D, k_loc, device="cuda", generator=g) * 0.02).bfloat16()
        f = timed(lambda: tp.gemm_rs(x, w), fc)
        n = timed(lambda: tp.gemm_rs_nccl(x, w), fc)
        loc = timed(lambda: plain_gemm(x, w), fc)
        rec(f"{name} {M}x{D}x{k_loc}", f, n, 2.0 * M * D * k_loc, (world - 1) / world * M * D * 2)
        out[-1]["local_gemm_ms"] = round(loc, 4)
        if rank == 0:
            print(json.dumps({"local_gemm_ms": round(loc, 4)}), flush=True)
    # ---- FSDP: the weight all-gather inside the GEMM that consumes it (ZeRO stage 3) --------
    # 1.3B shapes: x (M, 2048) against w_qkv (6208, 2048) gathered from row shards, with w_o
    # (2048, 2048) gathered by the same launch; the library composition all-gathers both
    # weights and then multiplies.
    import math

    from ..ops import _lib
    from .symm import SymmetricBuffer
    Dm = 2048
    for name, n_w, n_x in (("fsdp qkv (+w_o)", 6208, Dm * Dm), ("fsdp gate_up (+w_down)", 11264,
                                                               Dm * 5632)):
        if n_w % world or n_x % (8 * world) or a.only == "tp":
            continue
        wbuf = SymmetricBuffer(n_w * Dm * 2, fc.group)
        xbuf = SymmetricBuffer(n_x * 2, fc.group)
        w_full = wbuf.view(torch.bfloat16, n_w * Dm).view(n_w, Dm)
        w_full.normal_(0, 0.02, generator=g)
        e_full = xbuf.view(torch.bfloat16, n_x)
        xin = torch.randn(M, Dm, device="cuda", generator=g).bfloat16()
        rows_w = n_w // world
        blk = math.gcd(rows_w, 64)
        flags = torch.zeros(n_w // blk, dtype=torch.int32, device="cuda")
        outw = torch.empty(M, n_w, dtype=torch.bfloat16, device="cuda")
        calls = [0]
        st = _lib.status_word(torch.device("cuda", torch.cuda.current_device()))

        def fused():
            calls[0] += 1
            fc.device_barrier()   # every rank's shard is final (the optimizer's last barrier)
            _lib.check(_lib.lib().ceo_ag_gemm_bf16(
                wbuf.table(), 2, xin.data_ptr(), outw.data_ptr(), M, n_w, Dm, Dm, n_w, 0, 0, 0, 1.0,
                None, 0, flags.data_ptr(), calls[0], rank, world, -1, blk, xbuf.table(),
                n_x * 2 // world, st.data_ptr(), _lib.stream()), "ceo_ag_gemm_bf16")

        def nccl():
            sw = w_full[rank * rows_w:(rank + 1) * rows_w]
            dist.all_gather_into_tensor(w_full, sw)
            ne = n_x // world
            dist.all_gather_into_tensor(e_full, e_full[rank * ne:(rank + 1) * ne])
            plain_gemm(xin, w_full)
        f = timed(fused, fc)
        n = timed(nccl, fc)
        loc = timed(lambda: plain_gemm(xin, w_full), fc)
        rec(f"{name} {M}x{n_w}x{Dm}", f, n, 2.0 * M * n_w * Dm,
            (world - 1) / world * (n_w * Dm + n_x) * 2)
        out[-1]["local_gemm_ms"] = round(loc, 4)
        if rank == 0:
            print(json.dumps({"local_gemm_ms": round(loc, 4)}), flush=True)
        torch.cuda.synchronize()
        fc.barrier()
        wbuf.close()
        xbuf.close()
    tp.close()
    fc.close()
    if a.json and rank == 0:
        open(a.json, "w").write(json.dumps(out, indent=1))
    Comm().barrier()


if __name__ == "__main__":
    main()
