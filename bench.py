"""Headline benchmark: training tokens/s of EFLA-1.3B (configs/efla_1p3b.yaml) on N GPUs
of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A step is one optimizer step over the configured global batch (256 sequences of 4096
tokens = 1M tokens, fixed as N grows: strong scaling), run as micro-batches with fp32
gradient accumulation, then gradient reduce-scatter, AdamW on the sharded fp32 master
weights and parameter all-gather.  Tokens are seeded Zipf(1.1) over the vocabulary and the
weights N(0, 0.02): synthetic data, random initialisation.

Two timed regions, each bracketed by a barrier and a device synchronise, timed with CUDA
events, max over ranks: (1) `value`: K steps with the step's inputs already on the device;
(2) `e2e`: K steps through ``TrainEngine.train_step`` with the inputs in pinned host
memory (copied host->device inside the step) and the loss read back to the host every
step.  Every micro-batch streams far more than L2 (126 MB) through the device, so no
explicit L2 flush is needed between timed iterations.

``--impl reference`` times the reference's own CUDA kernels (``baseline/ref_step_bench.py``:
a kernel-sum floor of its step; the reference itself cannot run a training step) and prints
the same JSON line with ``"impl": "reference"``, or its ``unavailable`` line when the
reference's kernel library has not been built.

Every step reads fresh synthetic batches (the token stream never repeats within a run), so
``final_loss`` is a training loss, not the memorisation of one batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="ceo_clocks_", suffix=".csv")
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                power.append(float(p[3]))
            except ValueError:
                continue
            for nme, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nme)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        busy = [s for s, w in zip(sm, power) if w > 300] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "power_w_max": max(power) if power else None, "samples": len(sm)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "efla_1p3b.yaml"))
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per micro-batch")
    ap.add_argument("--global-batch", type=int, default=0, help="sequences per step (all GPUs)")
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--fp8", action="store_true",
                    help="side measurement, never the headline: forward projections on e4m3 "
                         "operands (training.fp8_training); reported with dtype bf16+fp8-forward")
    ap.add_argument("--fp8-dgrad", action="store_true",
                    help="--fp8 plus the projections' data gradients on e5m2 x e4m3 operands")
    ap.add_argument("--fp8-all", action="store_true",
                    help="--fp8-dgrad plus the weight gradients on e5m2 x e4m3 operands")
    ap.add_argument("--fp8-margin", type=int, default=-1,
                    help="FP8 scales leave 2^margin of headroom above the recorded amax "
                         "(-1: the engine's default, 2)")
    ap.add_argument("--tp", type=int, default=0,
                    help="tensor-parallel size (0: 1 for the default config, else the config's)")
    ap.add_argument("--cp", type=int, default=0, help="context-parallel size (0: the config's)")
    ap.add_argument("--zero-stage", type=int, default=-1,
                    help="ZeRO stage of the data-parallel replicas (1: one fused reduce-scatter + "
                         "update + all-gather kernel after backward; 2: bucket reduce-scatter "
                         "overlapped with backward; 3: + weight all-gather inside the consuming "
                         "GEMMs; -1: the config's runtime.zero_stage)")
    a = ap.parse_args(argv)

    if a.impl == "reference":
        # the reference's own kernels only: nothing of this framework's ops, models or engine
        from baseline import ref_step_bench
        try:
            rec = ref_step_bench.run(a.config, a.gpus, a.steps, a.warmup)
        except Exception as e:  # noqa: BLE001
            rec = ref_step_bench.unavailable(f"reference kernels failed: {type(e).__name__}: {e}"
                                             .replace("\n", " ")[:300])
            if int(os.environ.get("RANK", "0")) != 0:
                rec = {}
        if rec:
            print(json.dumps(rec))
        return 0

    import torch
    from ceo_b200.data.synthetic import SyntheticTokens
    from ceo_b200.ops import _lib
    from ceo_b200.parallel.comm import Comm, init_distributed
    from ceo_b200.runtime.engine import TrainEngine
    from ceo_b200.utils.config import Config

    rank, world, local = init_distributed()
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE is {world}: launch with torchrun")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        if a.comm in ("auto", "fused"):
            try:
                from ceo_b200.parallel.fused import FusedComm
                comm = FusedComm()
            except Exception as e:  # noqa: BLE001
                if a.comm == "fused":
                    raise
                if rank == 0:
                    print(f"[bench] fused collectives unavailable ({e}); using NCCL",
                          file=sys.stderr)
        if comm is None:
            comm = Comm()

    cfg = Config.parse_from_file(a.config)
    cfg.runtime.world_size = world
    headline = os.path.basename(a.config) == "efla_1p3b.yaml"
    tp = a.tp or (1 if headline else min(cfg.runtime.tensor_parallel_size, world))
    cp = a.cp or min(cfg.runtime.context_parallel_size, world)
    cfg.runtime.tensor_parallel_size, cfg.runtime.context_parallel_size = tp, cp
    dp = world // (tp * cp)
    seq = a.seq_len or cfg.data.seq_len
    cfg.data.seq_len = seq
    gbs = a.global_batch or cfg.training.global_batch_size
    mbs = a.micro_batch or cfg.training.micro_batch_size
    cfg.training.micro_batch_size = mbs
    cfg.training.fp8_training = bool(a.fp8 or a.fp8_dgrad or a.fp8_all)
    if a.zero_stage >= 0:
        cfg.runtime.zero_stage = a.zero_stage
    if cfg.training.fp8_training and cfg.runtime.zero_stage >= 3:
        cfg.runtime.zero_stage = 2  # the fused weight gather is a bf16 GEMM
    if world % (tp * cp) or gbs % (mbs * dp):
        raise SystemExit(f"global batch {gbs} is not a multiple of micro-batch {mbs} x dp {dp}")
    n_micro = gbs // (mbs * dp)
    tokens_per_step = gbs * seq

    if tp * cp > 1:
        # tensor / context parallel groups inside the node, data parallel (sharded optimizer)
        # across them; every rank of one tp x cp group reads the same batches
        from ceo_b200.runtime.parallel_engine import ParallelEngine
        eng = ParallelEngine(cfg, dev, fused=a.comm != "nccl" or tp > 1,
                             impl="nccl" if a.comm == "nccl" else "fused")
        data_rank = eng.pc.dp_rank
    else:
        eng = TrainEngine(cfg, dev, comm)
        if a.fp8_dgrad or a.fp8_all:
            eng.fp8.dgrad = True
        if a.fp8_all:
            eng.fp8.wgrad = True
        if eng.fp8 is not None and a.fp8_margin >= 0:
            eng.fp8.margin = a.fp8_margin
            for st in eng.fp8.states:
                for m in (st.x_meta, st.w_meta, st.g_meta):
                    m.margin = a.fp8_margin
        data_rank = rank
    data = SyntheticTokens(cfg.model.vocab_size, cfg.data.synthetic.kind or "zipf",
                           cfg.data.synthetic.s, cfg.data.synthetic.seed, data_rank)
    lr = cfg.training.learning_rate

    def fresh(n_steps, on_device):
        """n_steps x n_micro new micro-batches from the token stream (drawn before the timed
        region; pinned host memory, or already on the device)."""
        out = []
        for _ in range(n_steps):
            mb = [data.batch(mbs, seq, pin=True) for _ in range(n_micro)]
            out.append([(t.to(dev), g.to(dev)) for t, g in mb] if on_device else mb)
        return out

    def sync():
        if comm is not None:
            comm.barrier()
        torch.cuda.synchronize()

    for b in fresh(a.warmup, True):
        eng.train_step(b, lr)
    dev_batches = fresh(a.steps, True)
    host_batches = fresh(0 if a.skip_e2e else a.steps, False)
    sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- region 1: device-resident inputs ---------------------------------------------
    l0 = _lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for b in dev_batches:
        loss, gnorm = eng.train_step(b, lr)
    e1.record()
    sync()
    launches = _lib.launch_count - l0
    ms = e0.elapsed_time(e1)
    ms = comm.max_over_ranks(ms) if comm is not None else ms
    last_loss = float(loss)
    # ---- region 2: end to end through the public API ------------------------------------
    e2e = None
    if not a.skip_e2e:
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        e2.record()
        for b in host_batches:
            loss, gnorm = eng.train_step(b, lr)
            last_loss = loss.item()  # device -> host read of the step's result
        e3.record()
        sync()
        ms2 = e2.elapsed_time(e3)
        ms2 = comm.max_over_ranks(ms2) if comm is not None else ms2
        e2e = {"value": tokens_per_step * a.steps / (ms2 * 1e-3), "unit": "tokens/s",
               "ms_per_step": ms2 / a.steps,
               "h2d_bytes_per_step": sum(t.numel() * t.element_size() + g.numel() * g.element_size()
                                         for t, g in host_batches[0]) * world,
               "d2h_bytes_per_step": 4 * world}
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.read_status(dev)
    # what is partitioned over the data-parallel replicas: 0 nothing (one GPU), 1 optimizer
    # state, 2 + gradients (reduced bucket by bucket during backward), 3 + parameters (FSDP)
    zero_stage = getattr(eng, "zero_stage", 1 if dp > 1 else 0)
    shard = {0: f"dp{dp}", 1: f"zero1-dp{dp}", 2: f"zero2-dp{dp}", 3: f"fsdp{dp}"}[zero_stage]
    parallelism = shard if tp * cp == 1 else f"tp{tp}xcp{cp}x{shard}"
    peak_mem = torch.cuda.max_memory_allocated(dev)
    if comm is None:
        collectives = "none"
    elif not getattr(comm, "fused", False):
        collectives = "library collectives (NCCL)"
    else:
        collectives = "own kernels over NVLink peer memory: " + {
            1: "reduce-scatter + clip + AdamW + all-gather in one kernel after backward",
            2: "bucket reduce-scatter during backward, then norm + AdamW + all-gather in one kernel",
            3: "bucket reduce-scatter during backward, norm + AdamW in one kernel, weight "
               "all-gather inside the QKV and gate/up GEMMs"}.get(zero_stage, "fused optimizer step")
        if tp > 1:
            collectives += "; tensor parallel: all-gather -> GEMM and GEMM -> reduce-scatter kernels"
        if cp > 1:
            collectives += "; context parallel: in-kernel state exchange"
    if rank == 0:
        value = tokens_per_step * a.steps / (ms * 1e-3)
        flops = eng.model.flops_per_token(seq) * value
        out = {
            "metric": "train tokens/sec (box, device-timed, max over ranks) " + cfg.model.name,
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": ("bf16+fp8-forward+dgrad+wgrad" if a.fp8_all else
                      "bf16+fp8-forward+dgrad" if a.fp8_dgrad else
                      "bf16+fp8-forward" if a.fp8 else "bf16"),
            "data": "synthetic (seeded Zipf(1.1) tokens, N(0,0.02) random-init weights)",
            "config": {"model": cfg.model.name, "global_batch": gbs, "seq_len": seq,
                       "tokens_per_step": tokens_per_step, "micro_batch": mbs,
                       "grad_accum_steps": n_micro,
                       "parallelism": parallelism,
                       "zero_stage": zero_stage,
                       "optimizer": cfg.training.optimizer,
                       "collectives": collectives,
                       "l2": "inputs larger than L2 (each micro-batch streams >1 GB)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "model_tflops_per_gpu": flops / world / 1e12, "final_loss": last_loss,
            "wait_status": status, "impl": "ours",
            "torch_peak_alloc_gb": round(peak_mem / 2**30, 2),
        }
        print(json.dumps(out))
    if comm is not None:
        comm.barrier()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
