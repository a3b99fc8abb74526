"""Times the reference's own CUDA kernels (``baseline/_ref/libref_kernels.so``, built by
``baseline/build_ref_kernels.py``) against this framework's kernels on the same GPU, same
shapes: ``python baseline/ref_kernel_bench.py [--json out.json]``.

Each side is called through its public C entry point (the reference's ``*_cuda`` functions of
kernels/cuda/include/kernels.h; ours through ``ceo_b200.ops``), timed with CUDA events after
warm-up, L2 flushed before every timed call, median of the timed calls.  The reference's EFLA
kernels take q = k, one scalar beta, and keep bf16 state; ours is run in that same mode
(P = 2, no normalisation, scalar beta) on the same tensors.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from ceo_b200.ops import efla as E, matmul as G, nn as N  # noqa: E402
from ceo_b200.ops import _lib  # noqa: E402

CUDA_R_16BF = 14


def load_ref():
    p = os.path.join(HERE, "_ref", "libref_kernels.so")
    if not os.path.exists(p):
        raise SystemExit("build it first: python baseline/build_ref_kernels.py")
    lib = ctypes.CDLL(p)
    vp, sz, fl, it, bo = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_int, ctypes.c_bool
    sig = {
        "efla_forward_cuda": [vp, vp, vp, vp, sz, sz, sz, sz, fl, sz, vp],
        "efla_backward_cuda": [vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, fl, vp],
        "gemm_forward_cuda": [vp, vp, vp, vp, sz, sz, sz, it, it, it, vp],
        "rmsnorm_forward_cuda": [vp, vp, vp, sz, sz, fl, vp],
        "gelu_forward_cuda": [vp, vp, sz, bo, vp],
        "gelu_backward_cuda": [vp, vp, vp, sz, bo, vp],
        "adamw_step_cuda": [vp, vp, vp, vp, sz, fl, fl, fl, fl, fl, sz, vp],
        "lion_step_cuda": [vp, vp, vp, sz, fl, fl, fl, fl, vp],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, ctypes.c_int
    return lib


_flush = None


def time_ms(fn, iters=5, warmup=2):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=4096)
    a = ap.parse_args(argv)
    ref = load_ref()
    dev = "cuda"
    st = torch.cuda.current_stream().cuda_stream
    rows = []

    def rec(name, ref_ms, our_ms, note=""):
        r = {"kernel": name, "reference_ms": round(ref_ms, 4), "ours_ms": round(our_ms, 4),
             "speedup": round(ref_ms / our_ms, 2)}
        if note:
            r["note"] = note
        rows.append(r)
        print(json.dumps(r), flush=True)

    def ck(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} returned cudaError {rc}")

    # ---- EFLA forward / backward: B x T x 16 heads x 128 ----------------------------------
    B, T, H, d = a.batch, a.seq_len, 16, 128
    g = torch.Generator(device=dev).manual_seed(0)
    kv = (0.08 * torch.randn(B, T, 2, H, d, device=dev, generator=g)).bfloat16()
    k, v = kv[:, :, 0].contiguous(), kv[:, :, 1].contiguous()
    state = torch.zeros(B * H, d, d, device=dev, dtype=torch.bfloat16)
    out = torch.empty(B, T, H, d, device=dev, dtype=torch.bfloat16)

    def ref_fwd():
        state.zero_()
        ck(ref.efla_forward_cuda(k.data_ptr(), v.data_ptr(), state.data_ptr(), out.data_ptr(), B, T,
                                 H, d, 1.0, 64, st), "efla_forward_cuda")
    beta = torch.ones(1, device=dev)
    kvr = kv.clone().requires_grad_()
    rec(f"efla forward B{B} T{T} H{H} d{d}", time_ms(ref_fwd, 3, 1),
        time_ms(lambda: E.efla_qkv(kvr, beta, False), 5, 2),
        "reference: one CTA per (b,h), token-serial, bf16 state in global memory")
    go = torch.randn(B, T, H, d, device=dev, generator=g).bfloat16()
    gk, gv = torch.empty_like(k), torch.empty_like(v)
    gs = torch.empty_like(state)

    def ref_bwd():
        state.zero_()
        ck(ref.efla_backward_cuda(go.data_ptr(), k.data_ptr(), v.data_ptr(), state.data_ptr(),
                                  gk.data_ptr(), gv.data_ptr(), gs.data_ptr(), B, T, H, d, 1.0, st),
           "efla_backward_cuda")
    o, _ = E.efla_qkv(kvr, beta, False)
    rec("efla backward (same shape)", time_ms(ref_bwd, 3, 1),
        time_ms(lambda: torch.autograd.grad(o, kvr, go, retain_graph=True), 5, 2),
        f"reference allocates a {B * H * (T + 1) * d * d * 2 / 2**30:.1f} GiB state history "
        "inside the call and has no d(beta)")
    del kvr, o

    # ---- GEMM: the QKV projection of a 16k-token micro-batch --------------------------------
    M, K, Nn = 16384, 2048, 6144
    x = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w_in_out = (0.02 * torch.randn(K, Nn, device=dev, generator=g)).bfloat16()  # reference layout
    w_out_in = w_in_out.t().contiguous()
    c = torch.empty(M, Nn, device=dev, dtype=torch.bfloat16)
    rec(f"gemm forward {M}x{Nn}x{K}",
        time_ms(lambda: ck(ref.gemm_forward_cuda(x.data_ptr(), w_in_out.data_ptr(), None,
                                                 c.data_ptr(), M, K, Nn, CUDA_R_16BF, CUDA_R_16BF,
                                                 CUDA_R_16BF, st), "gemm_forward_cuda")),
        time_ms(lambda: G.gemm(x, w_out_in)),
        "reference: library GEMM with a handle created and destroyed per call")

    # ---- norms / activations ---------------------------------------------------------------
    D = 2048
    xn = torch.randn(M, D, device=dev, generator=g).bfloat16()
    wn = torch.ones(D, device=dev, dtype=torch.bfloat16)
    yn = torch.empty_like(xn)
    rec(f"rmsnorm forward {M}x{D}",
        time_ms(lambda: ck(ref.rmsnorm_forward_cuda(xn.data_ptr(), wn.data_ptr(), yn.data_ptr(),
                                                    M * D, D, 1e-6, st), "rmsnorm_forward_cuda")),
        time_ms(lambda: N.rmsnorm(xn, wn)))
    # rmsnorm_backward_cuda is deliberately not run: on this GPU it stops with "misaligned
    # address" (it adds a float atomically into the bf16 weight-gradient buffer through a
    # reinterpret cast, kernels/cuda/layernorm.cu:121-124, which is misaligned at odd indices).
    F = 5632
    xa = torch.randn(M, F, device=dev, generator=g).bfloat16()
    ya = torch.empty_like(xa)
    rec(f"gelu forward {M}x{F}",
        time_ms(lambda: ck(ref.gelu_forward_cuda(xa.data_ptr(), ya.data_ptr(), M * F, True, st),
                           "gelu_forward_cuda")),
        time_ms(lambda: N.activation(xa, "gelu")))

    # ---- optimizers on 2^27 parameters -------------------------------------------------------
    n = 1 << 27
    p16 = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    g16 = torch.randn(n, device=dev).bfloat16()
    m16, v16 = torch.zeros_like(p16), torch.zeros_like(p16)
    master, m32, v32 = (torch.zeros(n, device=dev) for _ in range(3))
    g32 = g16.float()
    L = _lib.lib()
    rec("adamw step, 2^27 parameters",
        time_ms(lambda: ck(ref.adamw_step_cuda(p16.data_ptr(), g16.data_ptr(), m16.data_ptr(),
                                               v16.data_ptr(), n, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, st),
                           "adamw_step_cuda")),
        time_ms(lambda: L.ceo_adamw_step(master.data_ptr(), m32.data_ptr(), v32.data_ptr(),
                                         g32.data_ptr(), 1, p16.data_ptr(), n, 1e-3, 0.9, 0.95, 1e-8,
                                         0.1, 1, None, 1.0, 0, st)),
        "reference keeps bf16 parameters and moments (10 B/param of traffic); ours keeps fp32 "
        "master + moments and writes the bf16 shadow (30 B/param)")
    rec("lion step, 2^27 parameters",
        time_ms(lambda: ck(ref.lion_step_cuda(p16.data_ptr(), g16.data_ptr(), m16.data_ptr(), n,
                                              1e-4, 0.95, 0.98, 0.1, st), "lion_step_cuda")),
        time_ms(lambda: L.ceo_lion_step(master.data_ptr(), m32.data_ptr(), g32.data_ptr(), 1,
                                        p16.data_ptr(), n, 1e-4, 0.95, 0.98, 0.1, None, 1.0, 0, st)),
        "reference: bf16 state (8 B/param); ours: fp32 master + momentum + bf16 shadow (22 B/param)")
    if a.json:
        open(a.json, "w").write(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
