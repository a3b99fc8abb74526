"""Worker for the multi-process CPU (gloo) tests: python dist_worker.py <what> <rank> <world> <port> <dir>."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ceo_b200.parallel.comm import Comm  # noqa: E402
from ceo_b200.runtime.engine import TrainEngine  # noqa: E402
from ceo_b200.runtime.fault import Heartbeat  # noqa: E402
from ceo_b200.utils import errors  # noqa: E402
from ceo_b200.utils.config import Config  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    what, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), \
        int(sys.argv[4]), sys.argv[5]
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime")
                          .timedelta(seconds=60))
    if what == "heartbeat":
        hb = Heartbeat(store, rank, world, interval=0.1, timeout=1.0).start()
        time.sleep(0.5)
        assert hb.dead_ranks() == []
        if rank == 1:       # rank 1 stops beating, then leaves between "steps"
            hb.pause()
            time.sleep(3.0)
            return
        t0 = time.time()
        while time.time() - t0 < 5:
            try:
                hb.check()
            except errors.RankFailure as e:
                open(os.path.join(out, f"detected{rank}"), "w").write(str(e))
                return
            time.sleep(0.1)
        raise SystemExit("failure not detected")
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    comm = Comm()
    if what == "collectives":
        t = torch.arange(8, dtype=torch.float32) + rank
        buf = t.clone()
        sl = comm.reduce_scatter(buf, rank * (8 // world), (rank + 1) * (8 // world))
        want = sum(torch.arange(8, dtype=torch.float32) + r for r in range(world))
        assert torch.equal(sl, want[rank * (8 // world):(rank + 1) * (8 // world)])
        full = torch.zeros(8)
        full[rank * (8 // world):(rank + 1) * (8 // world)] = rank + 1.0
        comm.all_gather(full, rank * (8 // world), (rank + 1) * (8 // world))
        assert full.tolist() == [float(i // (8 // world) + 1) for i in range(8)]
        a2a_in = torch.arange(world * 2, dtype=torch.float32) + 100 * rank
        a2a_out = torch.empty_like(a2a_in)
        comm.all_to_all(a2a_out, a2a_in)
        assert a2a_out.tolist() == [100.0 * r + 2 * rank + j for r in range(world) for j in range(2)]
        b = torch.tensor([float(rank)])
        comm.broadcast(b, src=world - 1)
        assert b.item() == world - 1
        assert comm.max_over_ranks(float(rank), device="cpu") == world - 1
        comm.barrier()
    elif what in ("zero_adamw", "zero_lion_muon"):
        cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
        cfg.training.optimizer = "adamw" if what == "zero_adamw" else "lion_muon"
        cfg.training.muon_iterations = 3
        cfg.runtime.world_size = world
        eng = TrainEngine(cfg, "cpu", comm, seed=0)
        g = torch.Generator().manual_seed(0)
        x = torch.randint(0, 256, (world * 2, 65), generator=g)
        mine = x[rank * 2:(rank + 1) * 2]
        for _ in range(3):
            loss, gn = eng.train_step([(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())], lr=1e-3)
        torch.save({"params": eng.flat.params.clone(), "loss": float(loss), "gn": float(gn)},
                   os.path.join(out, f"{what}_{rank}.pt"))
    elif what == "pipeline":
        from ceo_b200.models.model import EflaLM
        from ceo_b200.parallel.pipeline import PipelineRunner, PipelineStage, stage_bounds
        cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
        m = cfg.model
        m.num_layers = 3          # uneven split: stage 0 takes two layers
        stage = PipelineStage(m, "cpu", rank, world, seed=0, dtype=torch.float32)
        runner = PipelineRunner(stage)
        g = torch.Generator().manual_seed(1)
        x = torch.randint(0, m.vocab_size, (3, 2, 65), generator=g)   # three micro-batches
        batches = [(b[:, :-1].contiguous(), b[:, 1:].contiguous()) for b in x]
        loss = runner.run(batches)
        runner.sync_tied_grads()
        full = EflaLM(m, "cpu", dtype=torch.float32, seed=0)
        ref = sum(full(t, y) for t, y in batches) / len(batches)
        ref.backward()
        assert abs(float(loss) - float(ref)) < 1e-5, (float(loss), float(ref))
        lo, hi = stage_bounds(m.num_layers, world, rank)
        assert (lo, hi) == ((0, 2) if rank == 0 else (2, 3))
        for i, blk in enumerate(stage.blocks):
            for (n1, p1), (n2, p2) in zip(blk.named_parameters(),
                                          full.blocks[lo + i].named_parameters()):
                if p2.grad is None:
                    continue
                assert torch.allclose(p1.grad, p2.grad, atol=2e-5, rtol=1e-4), n1
        if stage.embed_tokens is not None:
            assert torch.allclose(stage.embed_tokens.grad, full.embed_tokens.grad, atol=2e-5,
                                  rtol=1e-4)
    elif what == "pipeline_trainer":
        # `train` with runtime.pipeline_parallel_size = 2: the Trainer builds the pipeline
        # engine, trains, and writes a checkpoint whose stages' tensors merge into one model
        from ceo_b200.runtime.checkpoint import CheckpointManager
        from ceo_b200.runtime.parallel_engine import PipelineEngine
        from ceo_b200.runtime.trainer import Trainer
        cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
        cfg.model.num_layers = 3
        cfg.runtime.world_size, cfg.runtime.pipeline_parallel_size = world, 2
        cfg.training.total_steps, cfg.training.global_batch_size = 4, 8
        cfg.training.micro_batch_size, cfg.checkpoint.save_interval = 4, 2
        cfg.checkpoint.async_save = False
        tr = Trainer(cfg, "cpu", checkpoint_dir=os.path.join(out, "ck"))
        assert isinstance(tr.engine, PipelineEngine) and tr.dp_world == world // 2
        res = tr.run()
        assert res["step"] == 4 and res["loss"] == res["loss"]
        dist.barrier()
        path = tr.ckpt.path_for(4)
        assert CheckpointManager.validate(path) == [], CheckpointManager.validate(path)
        merged = CheckpointManager.load_tensors(path)
        mine = {k: v[0] for k, v in tr.engine.model.state_dict_shards().items()}
        for k, v in mine.items():
            assert torch.equal(merged[k], v), k
        assert {f"blocks.{i}.mlp_down.weight" for i in range(3)} <= set(merged)
        if rank == 0:
            torch.save({"loss": res["loss"]}, os.path.join(out, "pp_done.pt"))
    comm.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
