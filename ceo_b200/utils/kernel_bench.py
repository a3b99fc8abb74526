"""Per-kernel timings against the measured roofline: ``python -m ceo_b200.utils.kernel_bench``.

Each kernel is timed with CUDA events on the launching stream after warm-up, with an L2
flush (a write of a buffer larger than L2) before every timed launch, and reported as
the median of the timed launches.  The denominators are the measured copy bandwidth and
library bf16 GEMM throughput in ``MEASURED_PEAKS.json`` at the repository root when that
file exists ("of measured"), else 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
``--torch`` also times the PyTorch/library op of the same shape for comparison.
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch

from ..ops import matmul as G, nn as N


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_flush = None


def time_ms(fn, iters=10, warmup=3):
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
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=5632)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--torch", action="store_true")
    ap.add_argument("--only", default="", help="run only the rows whose group name contains this")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--json", type=str, default="")
    a = ap.parse_args(argv)
    bw, fl, kind = peaks()
    dev = "cuda"
    M, D, Fh = a.tokens, a.d_model, a.ffn
    rows = []

    def rec(name, ms, flops=0.0, bytes_=0.0, base_ms=None):
        r = {"kernel": name, "ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r[f"frac_of_{kind}_gemm_peak"] = round(flops / (ms * 1e-3) / fl, 3)
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r[f"frac_of_{kind}_hbm"] = round(bytes_ / (ms * 1e-3) / bw, 3)
        if base_ms is not None:
            r["torch_ms"] = round(base_ms, 4)
        rows.append(r)
        print(json.dumps(r), flush=True)

    global time_ms
    _time = time_ms
    time_ms = lambda fn, iters=a.iters, warmup=3: _time(fn, iters, warmup)  # noqa: E731
    want = lambda group: (not a.only) or a.only in group  # noqa: E731
    x = torch.randn(M, D, device=dev).bfloat16()
    for name, n_out, k_in in (("qkv", 3 * D, D), ("gate_up", 2 * Fh, D), ("down", D, Fh),
                              ("out", D, D)):
        if not want("gemm_" + name):
            continue
        xin = x if k_in == D else torch.randn(M, k_in, device=dev).bfloat16()
        w = (torch.randn(n_out, k_in, device=dev) * 0.02).bfloat16()
        dy = torch.randn(M, n_out, device=dev).bfloat16()
        mg = torch.zeros(n_out, k_in, device=dev)
        fl_ = 2.0 * M * n_out * k_in
        tb = time_ms(lambda: xin @ w.t()) if a.torch else None
        rec(f"gemm_fwd_{name} {M}x{n_out}x{k_in}", time_ms(lambda: G.gemm(xin, w)), fl_, 0, tb)
        tb = time_ms(lambda: dy @ w) if a.torch else None
        rec(f"gemm_dgrad_{name}", time_ms(lambda: G.gemm(dy, w, b_mn=True)), fl_, 0, tb)
        tb = time_ms(lambda: mg.addmm_(dy.t().float(), xin.float())) if False else None
        tb = time_ms(lambda: dy.t() @ xin) if a.torch else None
        rec(f"gemm_wgrad_{name} (fp32 accumulate)",
            time_ms(lambda: G.gemm(dy, xin, a_mn=True, b_mn=True, out=mg, accumulate=True)),
            fl_, 0, tb)

    if want("fp8"):
        # forward projections on e4m3 operands; flops / time is compared with the bf16 peak
        from ..ops import fp8 as F8
        for name, n_out, k_in in (("qkv", 3 * D, D), ("gate_up", 2 * Fh, D), ("down", D, Fh)):
            xin = torch.randn(M, k_in, device=dev).bfloat16()
            w = (torch.randn(n_out, k_in, device=dev) * 0.02).bfloat16()
            mx, mw = F8.Fp8Meta(dev), F8.Fp8Meta(dev)
            xq, wq = F8.quantize(xin, mx), F8.quantize(w, mw)
            rec(f"fp8_quantize {M}x{k_in}", time_ms(lambda: F8.quantize(xin, mx)), 0,
                3.0 * M * k_in)
            rec(f"gemm_fp8_fwd_{name} {M}x{n_out}x{k_in}",
                time_ms(lambda: F8.gemm_fp8(xq, wq, mx, mw)), 2.0 * M * n_out * k_in)
            # gradients: e5m2 dy against e4m3 W^T (data) and e5m2 dy^T against e4m3 x^T (weight,
            # accumulated into an fp32 buffer), operands from the transposing quantiser
            dy = torch.randn(M, n_out, device=dev).bfloat16()
            mg_, mgrad = F8.Fp8Meta(dev, F8.E5M2), torch.zeros(n_out, k_in, device=dev)
            dyq, dyqt = F8.quantize_t(dy, mg_)
            _, xqt = F8.quantize_t(xin, mx)
            wtq = F8.quantize(w.t().contiguous(), mw)
            rec(f"fp8_quantize_t (codes + transposed codes) {M}x{n_out}",
                time_ms(lambda: F8.quantize_t(dy, mg_)), 0, 4.0 * M * n_out)
            rec(f"gemm_fp8_dgrad_{name}", time_ms(lambda: F8.gemm_fp8(dyq, wtq, mg_, mw)),
                2.0 * M * n_out * k_in)
            rec(f"gemm_fp8_wgrad_{name} (fp32 accumulate)",
                time_ms(lambda: F8.gemm_fp8(dyqt, xqt, mg_, mx, out=mgrad, accumulate=True)),
                2.0 * M * n_out * k_in)
    if want("norm"):
        w = torch.ones(D, device=dev).bfloat16().requires_grad_()
        xr = x.clone().requires_grad_()
        rec("rmsnorm_fwd", time_ms(lambda: N.rmsnorm(x, w)), 0, 2.0 * M * D * 2,
            time_ms(lambda: torch.nn.functional.rms_norm(x, (D,), w)) if a.torch else None)
        y, _ = N.rmsnorm(xr, w)
        dy = torch.randn_like(y)
        rec("rmsnorm_bwd", time_ms(lambda: torch.autograd.grad(y, (xr, w), dy, retain_graph=True)),
            0, 3.0 * M * D * 2)
        # the forms the transformer block uses: residual add fused into the forward kernel
        # (x, residual in; h, y out), residual stream's gradient added in the backward kernel
        r2 = torch.randn_like(x)
        rec("rmsnorm_fwd (+ residual)", time_ms(lambda: N.rmsnorm(x, w, residual=r2)), 0,
            4.0 * M * D * 2)
        y2, h2 = N.rmsnorm(xr, w, skip=True)
        dh = torch.randn_like(y)
        rec("rmsnorm_bwd (+ residual gradient)",
            time_ms(lambda: torch.autograd.grad((y2, h2), (xr, w), (dy, dh), retain_graph=True)),
            0, 4.0 * M * D * 2)
    if want("swiglu"):
        gu = torch.randn(M, 2 * Fh, device=dev).bfloat16().requires_grad_()
        rec("swiglu_fwd", time_ms(lambda: N.swiglu(gu)), 0, 3.0 * M * Fh * 2)
        o = N.swiglu(gu)
        do = torch.randn_like(o)
        rec("swiglu_bwd", time_ms(lambda: torch.autograd.grad(o, gu, do, retain_graph=True)), 0,
            5.0 * M * Fh * 2)
    if want("swiglu"):
        # the same two ops inside the GEMM epilogues (what the MLP runs): compare the pair
        # (plain GEMM + SwiGLU kernel) with the one fused launch
        w_up = (torch.randn(2 * Fh, D, device=dev) * 0.02).bfloat16()
        w_dn = (torch.randn(D, Fh, device=dev) * 0.02).bfloat16()
        gu_b = torch.empty(M, 2 * Fh, device=dev, dtype=torch.bfloat16)
        act_b = torch.empty(M, Fh, device=dev, dtype=torch.bfloat16)
        dy_b = torch.randn(M, D, device=dev).bfloat16()
        dgu_b = torch.empty_like(gu_b)
        rec(f"gemm_fwd_gate_up + SwiGLU epilogue {M}x{2 * Fh}x{D}",
            time_ms(lambda: G._gemm_swiglu(x, w_up, gu_b, M, 2 * Fh, D, False, 1, act_b)),
            2.0 * M * 2 * Fh * D)
        rec(f"gemm_dgrad_down + SwiGLU backward epilogue {M}x{Fh}x{D}",
            time_ms(lambda: G._gemm_swiglu(dy_b, w_dn, dgu_b, M, Fh, D, True, 2, gu_b)),
            2.0 * M * Fh * D)
    if want("efla"):
        from ..ops import efla as E
        from ..parallel.cp import efla_flops
        T, H, d = a.seq_len, a.heads, a.head_dim
        B = max(1, M // T)
        proj = (0.5 * torch.randn(B, T, 3 * H * d + 16, device=dev)).bfloat16().requires_grad_()
        rec(f"efla_fwd B{B} T{T} H{H} d{d} (prep + 3 kernels)",
            time_ms(lambda: E.efla_proj(proj, 3, H, d, True)), efla_flops(B, T, H, d, False))
        o, _ = E.efla_proj(proj, 3, H, d, True)
        do = torch.randn_like(o)
        rec("efla_bwd (3 kernels + prep)",
            time_ms(lambda: torch.autograd.grad(o, proj, do, retain_graph=True)),
            efla_flops(B, T, H, d, True) - efla_flops(B, T, H, d, False))
    if want("loss"):
        V = a.vocab
        hn = torch.randn(M, D, device=dev).bfloat16().requires_grad_()
        wh = (torch.randn(V, D, device=dev) * 0.02).bfloat16().requires_grad_()
        wh.main_grad = torch.zeros(V, D, device=dev)
        tgt = torch.randint(0, V, (M,), device=dev)
        rec(f"lm_head + cross-entropy fwd+bwd {M}x{V}x{D}",
            time_ms(lambda: N.linear_cross_entropy(hn, wh, tgt)), 6.0 * M * V * D)
    if want("optim"):
        n = 1 << 28
        ms_, m_, v_ = (torch.zeros(n, device=dev) for _ in range(3))
        g_ = torch.randn(n, device=dev)
        sh = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        from ..ops import _lib
        L = _lib.lib()
        rec("adamw (fp32 master + bf16 shadow) 2^28 elements",
            time_ms(lambda: L.ceo_adamw_step(ms_.data_ptr(), m_.data_ptr(), v_.data_ptr(),
                                             g_.data_ptr(), 1, sh.data_ptr(), n, 1e-3, 0.9, 0.95,
                                             1e-8, 0.1, 1, None, 1.0, 0, _lib.stream())), 0,
            n * 30.0)
    if a.json:
        Path(a.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
