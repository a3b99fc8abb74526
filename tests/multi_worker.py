"""Worker for the multi-GPU tests (launched with torchrun, one process per GPU)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ceo_b200.data.synthetic import SyntheticTokens  # noqa: E402
from ceo_b200.ops import _lib  # noqa: E402
from ceo_b200.parallel.comm import Comm, init_distributed  # noqa: E402
from ceo_b200.runtime.engine import TrainEngine  # noqa: E402
from ceo_b200.utils.config import Config  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_cfg(world):
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "efla_340m.yaml"))
    cfg.model.num_layers = 2
    cfg.model.vocab_size = 2048
    cfg.model.hidden_dim = 512
    cfg.model.num_heads = 8
    cfg.model.intermediate_dim = 1024
    cfg.runtime.world_size = world
    return cfg


def run_engine(comm, cfg, rank, steps=3, n_micro=1):
    eng = TrainEngine(cfg, torch.device("cuda", torch.cuda.current_device()), comm, seed=0)
    data = SyntheticTokens(cfg.model.vocab_size, "zipf", 1.1, 0, rank)
    losses = []
    for _ in range(steps):
        mbs = [tuple(t.cuda() for t in data.batch(2, 256)) for _ in range(n_micro)]
        loss, gn = eng.train_step(mbs, lr=1e-3)
        losses.append((float(loss), float(gn)))
    torch.cuda.synchronize()
    return eng, losses


def main():
    what = sys.argv[1]
    rank, world, local = init_distributed()
    torch.cuda.set_device(local)
    if what == "fused_vs_nccl":
        from ceo_b200.parallel.fused import FusedComm
        cfg = small_cfg(world)
        cfg.runtime.zero_stage = 1   # one fused kernel after the backward pass
        e_ref, l_ref = run_engine(Comm(), cfg, rank)
        fc = FusedComm()
        x = torch.arange(5, dtype=torch.float32, device="cuda") + rank
        got = fc.all_reduce_small(x)
        want = sum(torch.arange(5, dtype=torch.float32) + r for r in range(world))
        assert torch.allclose(got.cpu(), want), (got, want)
        fc.device_barrier()
        e_fus, l_fus = run_engine(fc, cfg, rank)
        for (a, ga), (b, gb) in zip(l_ref, l_fus):
            assert abs(a - b) < 2e-2 * abs(a) + 1e-3, (l_ref, l_fus)
            assert abs(ga - gb) < 2e-2 * abs(ga) + 1e-3, (l_ref, l_fus)
        pa, pb = e_ref.flat.params.float(), e_fus.flat.params.float()
        rel = ((pa - pb).norm() / pa.norm()).item()
        assert rel < 2e-3, rel
        # every rank must hold identical parameters after the fused all-gather
        chk = e_fus.flat.params.float().sum().reshape(1)
        allc = Comm().all_gather_cat(chk)
        assert torch.all(allc == allc[0]), allc
        assert float(e_fus.flat.grads.abs().max()) == 0.0
        assert _lib.read_status() == 0
        fc.close()
        if rank == 0:
            print("OK fused_vs_nccl", l_ref, l_fus, rel)
    elif what == "zero_stages":
        # ZeRO stage 1 / 2 / 3 on peer memory (one kernel after backward / bucket reductions
        # overlapped with backward / + weight all-gather inside the consuming GEMMs) against
        # the library composition (reduce-scatter, AdamW, all-gather) on the same data
        from ceo_b200.parallel.fused import FusedComm
        fc = FusedComm()
        cmp = Comm()
        for opt_kind in ("adamw", "lion"):
            cfg = small_cfg(world)
            cfg.training.optimizer = opt_kind
            # two micro-batches per step: gradients accumulate, the buckets leave during the
            # backward pass of the second one, the weight gather rides in the first forward
            e_ref, l_ref = run_engine(Comm(), cfg, rank, n_micro=2)
            assert e_ref.zero_stage == 1 and e_ref.flat.layout == "contiguous"
            for stage in ((1, 2, 3) if opt_kind == "adamw" else (2,)):
                cfg.runtime.zero_stage = stage
                eng, losses = run_engine(fc, cfg, rank, n_micro=2)
                assert eng.zero_stage == stage and eng.flat.layout == "segment"
                assert (len(eng.gathers) > 0) == (stage == 3)
                for (a, ga), (b, gb) in zip(l_ref, losses):
                    assert abs(a - b) < 2e-2 * abs(a) + 1e-3, (opt_kind, stage, l_ref, losses)
                    assert abs(ga - gb) < 2e-2 * abs(ga) + 1e-3, (opt_kind, stage, l_ref, losses)
                eng.materialize_params()
                for (n1, p1), (n2, p2) in zip(e_ref.model.named_parameters(),
                                              eng.model.named_parameters()):
                    if p1.numel() > 1:
                        rel = ((p1.float() - p2.float()).norm() / (p1.float().norm() + 1e-9)).item()
                        assert rel < (4e-3 if opt_kind == "adamw" else 2e-2), (opt_kind, stage, n1, rel)
                # identical parameters on every rank, gradients consumed
                chk = torch.stack([p.float().sum() for p in eng.model.parameters()]).sum().reshape(1)
                allc = cmp.all_gather_cat(chk)
                assert torch.all(allc == allc[0]), (stage, allc)
                assert float(eng.flat.grads.abs().max()) == 0.0
                assert _lib.read_status() == 0
        fc.close()
        if rank == 0:
            print("OK zero_stages")
    elif what == "tp_fused":
        from ceo_b200.parallel.fused import FusedComm
        from ceo_b200.parallel.tp import TPContext, column_parallel_linear, row_parallel_linear
        fc = FusedComm()
        M, K, N = 256 * world, 512, 768
        tp = TPContext(fc, M, max(K, N), copy_ctas=4)
        g = torch.Generator(device="cuda").manual_seed(0)
        x_full = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        w_col = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
        w_row = (torch.randn(K, N, device="cuda", generator=g) * 0.05).bfloat16()
        rows = M // world
        xs = x_full[rank * rows:(rank + 1) * rows].contiguous()
        for rep in range(5):   # repeated calls reuse flags / staging / counters
            if rep == 3:       # the last two through the copy-first mode of the all-gather
                tp.copy_ctas = -1
            y = tp.ag_gemm(xs, w_col)
            want = x_full.float() @ w_col.float().t()
            e1 = ((y.float() - want).norm() / want.norm()).item()
            assert e1 < 6e-3, ("ag_gemm", rep, e1)
            # row parallel: every rank holds a K-slice; emulate with rank-dependent inputs
            a_r = (x_full.float() * (1 + rank)).bfloat16()
            res = torch.randn(rows, N, device="cuda", generator=g).bfloat16()
            z = tp.gemm_rs(a_r, w_row.t().contiguous() if False else w_row, w_mn=True, residual=res)
            tot = sum((x_full.float() * (1 + r)).bfloat16().float() for r in range(world))
            want2 = (tot @ w_row.float())[rank * rows:(rank + 1) * rows] + res.float()
            e2 = ((z.float() - want2).norm() / want2.norm()).item()
            assert e2 < 1e-2, ("gemm_rs", rep, e2)
        # autograd: fused vs NCCL composition
        outs = {}
        for impl in ("nccl", "fused"):
            xs_l = xs.clone().requires_grad_()
            wc = w_col.clone().requires_grad_()
            wr = (torch.randn(K, N, device="cuda", generator=torch.Generator(device="cuda")
                              .manual_seed(5)) * 0.05).bfloat16().requires_grad_()
            h = column_parallel_linear(xs_l, wc, tp, impl)          # (M, N)
            o = row_parallel_linear(h, wr, tp, residual=xs_l, impl=impl)  # (rows, K)
            (o.float() * 0.01).sum().backward()
            outs[impl] = (o.detach().float(), xs_l.grad.float(), wc.grad.float(), wr.grad.float())
        for a, b in zip(outs["nccl"], outs["fused"]):
            rel = ((a - b).norm() / (a.norm() + 1e-9)).item()
            assert rel < 2e-2, rel
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        tp.close()
        fc.close()
        if rank == 0:
            print("OK tp_fused", e1, e2)
    elif what == "cp":
        from ceo_b200.ops import efla, reference as ref
        from ceo_b200.parallel.cp import CPContext, cp_delta_rule
        from ceo_b200.parallel.fused import FusedComm
        fc = FusedComm()
        B, Tl, H, d = 2, 128, 2, 128
        T = Tl * world
        cp = CPContext(fc, B * H, d)
        g = torch.Generator(device="cuda").manual_seed(3)     # same on all ranks: full tensors
        q = torch.randn(B, T, H, d, device="cuda", generator=g)
        k = torch.randn(B, T, H, d, device="cuda", generator=g)
        q = (q / q.norm(dim=-1, keepdim=True)).bfloat16()
        k = (k / k.norm(dim=-1, keepdim=True)).bfloat16()
        v = torch.randn(B, T, H, d, device="cuda", generator=g).bfloat16()
        alpha = -torch.expm1(-torch.sigmoid(torch.randn(B, T, H, device="cuda", generator=g)))
        do = torch.randn(B, T, H, d, device="cuda", generator=g).bfloat16()
        sl = slice(rank * Tl, (rank + 1) * Tl)
        for rep in range(2):
            loc = [t[:, sl].detach().clone().requires_grad_() for t in (q, k, v, alpha)]
            o = cp_delta_rule(*loc, cp)
            (o.float() * do[:, sl].float()).sum().backward()
            full = [t.detach().clone().requires_grad_() for t in (q, k, v, alpha)]
            of, _ = efla.delta_rule(*full)
            (of.float() * do.float()).sum().backward()
            rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
            errs = [rel(o, of[:, sl])] + [rel(a.grad, b.grad[:, sl]) for a, b in zip(loc, full)]
            assert max(errs) < 2e-2, errs
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        cp.close()
        fc.close()
        if rank == 0:
            print("OK cp", errs)
    elif what in ("tp_model", "cp_model"):
        from ceo_b200.runtime.parallel_engine import ParallelEngine
        cfg = small_cfg(world)
        cfg.model.num_heads = 4
        cfg.model.head_dim = 128
        # context parallel: every rank's span is at least one 64-token chunk
        seq = 256 if what == "tp_model" else max(256, 64 * world)
        cfg.data.seq_len = seq
        cfg.training.micro_batch_size = 2
        cfg.runtime.tensor_parallel_size = world if what == "tp_model" else 1
        cfg.runtime.context_parallel_size = world if what == "cp_model" else 1
        data = SyntheticTokens(cfg.model.vocab_size, "zipf", 1.1, 0, 0)   # same data on all ranks
        batches = [data.batch(2, seq) for _ in range(3)]
        par = ParallelEngine(cfg, torch.device("cuda", torch.cuda.current_device()))
        lp = [tuple(float(x) for x in par.train_step([b], lr=1e-3)) for b in batches]
        cfg1 = small_cfg(1)
        cfg1.model.num_heads, cfg1.model.head_dim = 4, 128
        single = TrainEngine(cfg1, torch.device("cuda", torch.cuda.current_device()), None, seed=0)
        ls = [tuple(float(x) for x in single.train_step([(t.cuda(), g.cuda())], lr=1e-3))
              for t, g in batches]
        for (a, ga), (b, gb) in zip(lp, ls):
            assert abs(a - b) < 3e-2 * abs(b), (lp, ls)
            assert abs(ga - gb) < 6e-2 * abs(gb), (lp, ls)
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        par.close()
        if rank == 0:
            print(f"OK {what}", lp, ls)
    elif what == "train_tp":
        # the Trainer (what `efla-train train` builds) on a tensor-parallel mesh from the
        # config: trains, saves a sharded checkpoint, and the merged tensors load into a
        # single-GPU model that gives the same loss
        import tempfile

        import torch.distributed as dist

        from ceo_b200.models.model import EflaLM
        from ceo_b200.runtime.checkpoint import CheckpointManager
        from ceo_b200.runtime.parallel_engine import ParallelEngine
        from ceo_b200.runtime.trainer import Trainer
        cfg = small_cfg(world)
        cfg.model.num_heads, cfg.model.head_dim = 4, 128
        cfg.data.seq_len = 256
        cfg.training.micro_batch_size, cfg.training.global_batch_size = 2, 4
        cfg.training.total_steps, cfg.checkpoint.save_interval = 2, 2
        cfg.checkpoint.async_save = False
        cfg.telemetry.metrics_interval = 1
        cfg.runtime.tensor_parallel_size = world
        box = [tempfile.mkdtemp() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        tr = Trainer(cfg, checkpoint_dir=box[0])
        assert isinstance(tr.engine, ParallelEngine) and tr.dp_world == 1
        res = tr.run()
        assert res["step"] == 2 and res["loss"] == res["loss"]
        dist.barrier()
        path = tr.ckpt.path_for(2)
        assert CheckpointManager.validate(path) == [], CheckpointManager.validate(path)
        merged = CheckpointManager.load_tensors(path)
        data = SyntheticTokens(cfg.model.vocab_size, "zipf", 1.1, 7, 0)
        tok, tgt = (t.cuda() for t in data.batch(2, 256))
        with torch.no_grad():
            lp = float(tr.engine.model(tok, tgt))
        lp_all = Comm().all_gather_cat(torch.tensor([lp], device="cuda"))
        single = EflaLM(cfg.model, "cuda", seed=99)
        single.load_reference_state(merged)
        with torch.no_grad():
            ls = float(single(tok, tgt))
        # each tensor-parallel rank scores its own row shard: their mean is the batch loss
        assert abs(float(lp_all.mean()) - ls) < 2e-2 * abs(ls), (lp_all, ls)
        tr2 = Trainer(cfg, checkpoint_dir=box[0])
        md = tr2.resume()
        assert md["step"] == 2 and tr2.engine.optimizer.step_count == 2
        for a, b in zip(tr.engine.model.parameters(), tr2.engine.model.parameters()):
            assert torch.equal(a, b)
        assert torch.equal(tr.engine.flat.buffer("exp_avg"), tr2.engine.flat.buffer("exp_avg"))
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        tr.engine.close()
        tr2.engine.close()
        if rank == 0:
            print("OK train_tp", lp_all.tolist(), ls)
    elif what == "pipeline":
        # two pipeline stages over NCCL point-to-point against the whole model on one GPU
        from ceo_b200.models.model import EflaLM
        from ceo_b200.parallel.pipeline import PipelineRunner, PipelineStage
        cfg = small_cfg(1)
        m = cfg.model
        m.num_heads, m.head_dim, m.num_layers = 4, 128, 3
        dev = torch.device("cuda", torch.cuda.current_device())
        stage = PipelineStage(m, dev, rank, world, seed=0)
        runner = PipelineRunner(stage)
        data = SyntheticTokens(m.vocab_size, "zipf", 1.1, 0, 0)
        batches = [tuple(t.to(dev) for t in data.batch(2, 256)) for _ in range(3)]
        loss = float(runner.run(batches))
        runner.sync_tied_grads()
        full = EflaLM(m, dev, seed=0)
        ref = sum(full(t, y) for t, y in batches) / len(batches)
        ref.backward()
        assert abs(loss - float(ref)) < 2e-2 * abs(float(ref)), (loss, float(ref))
        rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
        errs = []
        for i, blk in enumerate(stage.blocks):
            for (n1, p1), (n2, p2) in zip(blk.named_parameters(),
                                          full.blocks[stage.lo + i].named_parameters()):
                if p1.grad is not None and p2.grad is not None and p2.grad.abs().max() > 0:
                    errs.append(rel(p1.grad, p2.grad))
        assert errs and max(errs) < 5e-2, errs
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        if rank == 0:
            print("OK pipeline", loss, float(ref), max(errs))
    else:
        raise SystemExit(f"unknown test {what}")
    Comm().barrier()


if __name__ == "__main__":
    main()
