"""The reference arm of ``bench.py``: a kernel-sum floor of the reference's training step.

The reference cannot run a training step (its model forward rejects non-CPU devices, its
backward is a stub and it issues no collective), but its CUDA kernels build and run.  This
module loads ONLY ``baseline/_ref/libref_kernels.so`` (the reference's own ``.cu`` files,
compiled by ``baseline/build_ref_kernels.py``; nothing of this framework's kernels, models or
engine is imported), times the reference's public ``*_cuda`` entry points at the benchmark's
micro-batch shapes with CUDA events, and composes

    step = micro-batches x (layers x per-layer kernels + LM head GEMMs) + optimizer

That sum leaves out everything the reference has no kernel for (embedding, cross-entropy,
residual adds, gradient accumulation, every collective) and its RMSNorm backward, which
faulted on B200 ("misaligned address", kernels/cuda/layernorm.cu:121-124) and is not run
again: it is a LOWER bound on the reference's step time, so a ratio against it is
conservative.  The reference's kernels implement q = k with one scalar beta and a GELU MLP;
the GEMM shapes are the benchmark config's (fused q/k/v, gate/up, down, out), so the
floating-point work of the projections matches.

Entry points used: efla_forward_cuda / efla_backward_cuda (kernels/cuda/efla.cu:482,543),
gemm_forward_cuda / gemm_backward_cuda (gemm.cu:303,400), rmsnorm_forward_cuda
(layernorm.cu:307), gelu_forward_cuda / gelu_backward_cuda (layernorm.cu:385,405),
adamw_step_cuda (optim.cu:657).
"""
from __future__ import annotations

import ctypes
import json
import os
import statistics
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
if os.path.dirname(HERE) not in sys.path:
    sys.path.insert(0, os.path.dirname(HERE))
LIB = os.path.join(HERE, "_ref", "libref_kernels.so")
CUDA_R_16BF = 14

COMPOSITION = ("sum of the reference's own kernels at the benchmark's micro-batch shapes "
               "(per layer: rmsnorm_forward x2, gemm_forward + gemm_backward for qkv / out / "
               "gate-up / down, efla_forward + efla_backward, gelu_forward + gelu_backward; per "
               "micro-batch: LM-head gemm_forward + gemm_backward; per step: adamw_step over all "
               "parameters); no collectives, no embedding, no cross-entropy; "
               "rmsnorm_backward_cuda left out (it faulted on B200 and is not run again); "
               "q = k, scalar beta, GELU MLP")


def unavailable(reason: str) -> dict:
    return {"impl": "reference", "unavailable": reason}


def _load():
    lib = ctypes.CDLL(LIB)
    vp, sz, fl, it, bo = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_int, ctypes.c_bool
    sig = {
        "efla_forward_cuda": [vp, vp, vp, vp, sz, sz, sz, sz, fl, sz, vp],
        "efla_backward_cuda": [vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, fl, vp],
        "gemm_forward_cuda": [vp, vp, vp, vp, sz, sz, sz, it, it, it, vp],
        "gemm_backward_cuda": [vp, vp, vp, vp, vp, vp, sz, sz, sz, vp],
        "rmsnorm_forward_cuda": [vp, vp, vp, sz, sz, fl, vp],
        "gelu_forward_cuda": [vp, vp, sz, bo, vp],
        "gelu_backward_cuda": [vp, vp, vp, sz, bo, vp],
        "adamw_step_cuda": [vp, vp, vp, vp, sz, fl, fl, fl, fl, fl, sz, vp],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, ctypes.c_int
    return lib


def run(config_path: str, gpus: int, steps: int, warmup: int) -> dict:
    """Returns the JSON record of the reference arm (or its ``unavailable`` record)."""
    if not os.path.exists(LIB):
        return unavailable("baseline/_ref/libref_kernels.so has not been built "
                           "(python baseline/build_ref_kernels.py <reference tree>)")
    import torch
    import torch.distributed as dist
    from ceo_b200.utils.config import Config  # plain Python: the YAML schema only

    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != gpus:
        raise SystemExit(f"--gpus {gpus} but WORLD_SIZE is {world}: launch with torchrun")
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    st = torch.cuda.current_stream().cuda_stream
    ref = _load()

    cfg = Config.parse_from_file(config_path)
    m, t = cfg.model, cfg.training
    D, H, d, F, V, L = m.hidden_dim, m.num_heads, m.head_dim, m.intermediate_dim, m.vocab_size, \
        m.num_layers
    T, mbs, gbs = cfg.data.seq_len, t.micro_batch_size, t.global_batch_size
    n_micro = gbs // (mbs * world)
    M = mbs * T
    hd = H * d
    steps, warmup = max(1, steps), max(3, warmup)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > L2 (126 MB)

    def ck(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} returned cudaError {rc}")

    def time_ms(fn):
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16
    parts = {}

    # ---- EFLA recurrence (q = k, scalar beta, bf16 state in global memory) ----------------
    k = (0.08 * torch.randn(mbs, T, H, d, device=dev, generator=g)).to(bf)
    v = (0.08 * torch.randn(mbs, T, H, d, device=dev, generator=g)).to(bf)
    state = torch.zeros(mbs * H, d, d, device=dev, dtype=bf)
    out = torch.empty(mbs, T, H, d, device=dev, dtype=bf)
    go = torch.randn(mbs, T, H, d, device=dev, generator=g).to(bf)
    gk, gv, gs = torch.empty_like(k), torch.empty_like(v), torch.empty_like(state)

    def efla_fwd():
        state.zero_()
        ck(ref.efla_forward_cuda(k.data_ptr(), v.data_ptr(), state.data_ptr(), out.data_ptr(), mbs,
                                 T, H, d, 1.0, 64, st), "efla_forward_cuda")

    def efla_bwd():
        state.zero_()
        ck(ref.efla_backward_cuda(go.data_ptr(), k.data_ptr(), v.data_ptr(), state.data_ptr(),
                                  gk.data_ptr(), gv.data_ptr(), gs.data_ptr(), mbs, T, H, d, 1.0,
                                  st), "efla_backward_cuda")
    parts["efla_forward"] = time_ms(efla_fwd)
    parts["efla_backward"] = time_ms(efla_bwd)
    del k, v, out, go, gk, gv

    # ---- projections: the reference's library GEMM (handle created per call) --------------
    def gemm_pair(name, K_, N_):
        x = torch.randn(M, K_, device=dev, generator=g).to(bf)
        w = (0.02 * torch.randn(K_, N_, device=dev, generator=g)).to(bf)   # (in, out)
        y = torch.empty(M, N_, device=dev, dtype=bf)
        dy = torch.randn(M, N_, device=dev, generator=g).to(bf)
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        parts[name + "_forward"] = time_ms(lambda: ck(ref.gemm_forward_cuda(
            x.data_ptr(), w.data_ptr(), None, y.data_ptr(), M, K_, N_, CUDA_R_16BF, CUDA_R_16BF,
            CUDA_R_16BF, st), "gemm_forward_cuda"))
        parts[name + "_backward"] = time_ms(lambda: ck(ref.gemm_backward_cuda(
            dy.data_ptr(), x.data_ptr(), w.data_ptr(), dx.data_ptr(), dw.data_ptr(), None, M, K_,
            N_, st), "gemm_backward_cuda"))

    P = 3 if m.efla.use_query else 2
    gemm_pair("gemm_qkv", D, P * hd)
    gemm_pair("gemm_out", hd, D)
    gemm_pair("gemm_up", D, 2 * F if m.activation == "swiglu" else F)
    gemm_pair("gemm_down", F, D)
    gemm_pair("gemm_lm_head", D, V)

    # ---- norms and activations -------------------------------------------------------------
    xn = torch.randn(M, D, device=dev, generator=g).to(bf)
    wn = torch.ones(D, device=dev, dtype=bf)
    yn = torch.empty_like(xn)
    parts["rmsnorm_forward"] = time_ms(lambda: ck(ref.rmsnorm_forward_cuda(
        xn.data_ptr(), wn.data_ptr(), yn.data_ptr(), M * D, D, 1e-6, st), "rmsnorm_forward_cuda"))
    xa = torch.randn(M, F, device=dev, generator=g).to(bf)
    ya, da = torch.empty_like(xa), torch.empty_like(xa)
    parts["gelu_forward"] = time_ms(lambda: ck(ref.gelu_forward_cuda(
        xa.data_ptr(), ya.data_ptr(), M * F, True, st), "gelu_forward_cuda"))
    parts["gelu_backward"] = time_ms(lambda: ck(ref.gelu_backward_cuda(
        ya.data_ptr(), xa.data_ptr(), da.data_ptr(), M * F, True, st), "gelu_backward_cuda"))
    del xn, yn, xa, ya, da

    # ---- optimizer: bf16 parameters and moments, every parameter of the model --------------
    n_params = V * D * (1 if m.tie_embeddings else 2) + L * (
        P * hd * D + hd * D + (2 * F if m.activation == "swiglu" else F) * D + F * D + 2 * D) + D
    p16 = torch.zeros(n_params, device=dev, dtype=bf)
    g16 = torch.randn(n_params, device=dev).to(bf)
    m16, v16 = torch.zeros_like(p16), torch.zeros_like(p16)
    parts["adamw_step"] = time_ms(lambda: ck(ref.adamw_step_cuda(
        p16.data_ptr(), g16.data_ptr(), m16.data_ptr(), v16.data_ptr(), n_params, 1e-3, 0.9, 0.95,
        1e-8, 0.1, 1, st), "adamw_step_cuda"))

    per_layer = (2 * parts["rmsnorm_forward"] + parts["efla_forward"] + parts["efla_backward"]
                 + parts["gelu_forward"] + parts["gelu_backward"]
                 + sum(parts[f"gemm_{n}_{d_}"] for n in ("qkv", "out", "up", "down")
                       for d_ in ("forward", "backward")))
    per_micro = L * per_layer + parts["gemm_lm_head_forward"] + parts["gemm_lm_head_backward"]
    step_ms = n_micro * per_micro + parts["adamw_step"]
    if world > 1:
        tmax = torch.tensor([step_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        step_ms = float(tmax)
    tokens_per_step = gbs * T
    rec = {
        "metric": "train tokens/sec (box, device-timed, max over ranks) " + m.name,
        "value": tokens_per_step / (step_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded normal tensors of the benchmark's shapes)",
        "config": {"model": m.name, "global_batch": gbs, "seq_len": T,
                   "tokens_per_step": tokens_per_step, "micro_batch": mbs,
                   "grad_accum_steps": n_micro, "parallelism": f"dp{world} without collectives",
                   "optimizer": "adamw (bf16 state)",
                   "l2": "256 MB buffer written before every timed call"},
        "impl": "reference", "composition": COMPOSITION, "same_config": False,
        # ms_per_step is COMPOSED from the per-kernel medians below (the full step would take
        # minutes per iteration); timed_kernel_calls says how much was actually run and timed
        "composed": True, "timed_kernel_calls": steps * len(parts),
        "kernel_ms": {k_: round(v_, 4) for k_, v_ in parts.items()},
    }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return rec if rank == 0 else {}


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(os.path.dirname(HERE), "configs",
                                                     "efla_1p3b.yaml"))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    r = run(a.config, a.gpus, a.steps, a.warmup)
    if r:
        print(json.dumps(r))
