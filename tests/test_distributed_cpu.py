"""Multi-process CPU tests (gloo, world_size 2): collectives, ZeRO-sharded optimizers equal
to the single-process result, heartbeat-based failure detection, recovery driver."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from ceo_b200.runtime import fault
from ceo_b200.runtime.engine import TrainEngine
from ceo_b200.utils import errors
from ceo_b200.utils.config import Config

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(what, world, out, timeout=240):
    port = _port()
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker.py"), what, str(r),
                               str(world), str(port), str(out)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append((p.returncode, o))
    for rc, o in outs:
        assert rc == 0, o[-3000:]


def test_gloo_collectives(tmp_path):
    _spawn("collectives", 2, tmp_path)


@pytest.mark.parametrize("kind", ["zero_adamw", "zero_lion_muon"])
def test_sharded_optimizer_matches_single_process(tmp_path, kind):
    world = 2
    _spawn(kind, world, tmp_path)
    res = [torch.load(tmp_path / f"{kind}_{r}.pt") for r in range(world)]
    assert torch.equal(res[0]["params"][:1000], res[1]["params"][:1000])
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
    cfg.training.optimizer = "adamw" if kind == "zero_adamw" else "lion_muon"
    cfg.training.muon_iterations = 3
    eng = TrainEngine(cfg, "cpu", None, seed=0)
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 256, (world * 2, 65), generator=g)
    for _ in range(3):
        # one process, the two ranks' micro-batches as gradient accumulation: with the
        # optimizer's 1/n_micro scale the summed gradient matches sum-over-ranks / world
        batches = [(x[r * 2:(r + 1) * 2, :-1].contiguous(), x[r * 2:(r + 1) * 2, 1:].contiguous())
                   for r in range(world)]
        loss, gn = eng.train_step(batches, lr=1e-3)
    n = eng.flat.numel()
    ref_params = eng.flat.params[:n]
    assert torch.allclose(res[0]["params"][:n], ref_params, atol=2e-5), \
        (res[0]["params"][:n] - ref_params).abs().max()


def test_pipeline_1f1b_matches_whole_model(tmp_path):
    """Two pipeline stages over gloo: loss and every gradient equal the single-process model."""
    _spawn("pipeline", 2, tmp_path)


def test_heartbeat_detects_silent_rank(tmp_path):
    _spawn("heartbeat", 2, tmp_path, timeout=60)
    msg = (tmp_path / "detected0").read_text()
    assert "rank(s) [1]" in msg


def test_kernel_watch_and_step_guard():
    state = {"code": 0}
    kw = fault.KernelWatch(lambda: state["code"], lambda: state.update(code=0))
    kw.check()
    state["code"] = 112
    with pytest.raises(errors.KernelWaitTimeout, match="peer barrier 1: no signal from rank 2"):
        kw.check()
    assert state["code"] == 0
    assert "MMA waiting for data" in fault.describe_status(2)
    g = fault.StepGuard(None, kw)
    assert g.run(lambda: (1.5, 0.1)) == (1.5, 0.1)
    with pytest.raises(errors.NaNDetected):
        g.run(lambda: (float("nan"), 0.0))
    with pytest.raises(errors.CommunicationError):
        g.run(lambda: (_ for _ in ()).throw(RuntimeError("NCCL communicator was aborted")))
    with pytest.raises(RuntimeError, match="other"):
        g.run(lambda: (_ for _ in ()).throw(RuntimeError("other")))


def test_run_with_recovery_resumes_after_injected_failure(tmp_path):
    from ceo_b200.runtime.trainer import Trainer
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
    cfg.data.seq_len = 32
    cfg.training.global_batch_size = cfg.training.micro_batch_size = 2
    cfg.checkpoint.save_interval = 2
    cfg.checkpoint.async_save = False
    inj = fault.FaultInjector()
    inj.fail_at_step = 5
    restarts = []

    def make(attempt):
        tr = Trainer(cfg, "cpu", checkpoint_dir=str(tmp_path / "ck"))
        orig = tr.engine.train_step

        def guarded(batches, lr=None):
            inj.maybe_raise(tr.engine.step_count + 1)
            return orig(batches, lr)
        tr.engine.train_step = guarded
        return tr
    tr = fault.run_with_recovery(make, total_steps=8, on_restart=lambda a, e: restarts.append(str(e)))
    assert tr.engine.step_count == 8 and restarts == ["injected failure"]
    assert tr.ckpt.list_checkpoints()[-1] == 8
    # a corrupted newest checkpoint falls back to the one before it
    fault.FaultInjector.corrupt_file(os.path.join(tr.ckpt.path_for(8), "tensors.bin"))
    tr2 = fault.run_with_recovery(lambda a: Trainer(cfg, "cpu", checkpoint_dir=str(tmp_path / "ck")),
                                  total_steps=8)
    assert tr2.engine.step_count == 8


def test_train_command_builds_pipeline_engine_and_merged_checkpoint(tmp_path):
    """runtime.pipeline_parallel_size = 2 on two gloo ranks: Trainer -> PipelineEngine, a
    checkpoint written stage by stage that reads back as ONE model - also by a single-process
    run of the same config without pipeline stages."""
    _spawn("pipeline_trainer", 2, tmp_path)
    assert (tmp_path / "pp_done.pt").exists()
    from ceo_b200.runtime.trainer import Trainer
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
    cfg.model.num_layers = 3
    cfg.training.total_steps, cfg.training.global_batch_size = 6, 8
    cfg.training.micro_batch_size = 4
    cfg.checkpoint.save_interval = 0
    tr = Trainer(cfg, "cpu", checkpoint_dir=str(tmp_path / "ck"))
    md = tr.resume()   # pipeline size 2 -> 1: parameters load, the moments restart
    assert md["step"] == 4 and tr.engine.step_count == 4
    res = tr.run()
    assert res["step"] == 6 and res["loss"] == res["loss"]


def test_tensor_parallel_checkpoint_shards_merge_and_reload(tmp_path):
    """Tensor-parallel ranks write their slices; the merged view equals the single-GPU model
    drawn from the same seed, and loads at another tensor-parallel size."""
    from types import SimpleNamespace

    from ceo_b200.models.model import EflaLM
    from ceo_b200.models.parallel_model import ParallelEflaLM
    from ceo_b200.runtime.checkpoint import CheckpointManager
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
    m = cfg.model
    full = EflaLM(m, "cpu", dtype=torch.bfloat16, seed=3).state_dict_reference()
    for r in reversed(range(2)):
        pm = ParallelEflaLM(m, "cpu", tp=SimpleNamespace(rank=r, world=2), seed=3)
        CheckpointManager(tmp_path / "ck", rank=r, world=2).save(
            7, {}, {}, None, tensor_shards=pm.state_dict_shards(), shard_rank=r, shard_world=2,
            shard_timeout=5.0)
    path = str(tmp_path / "ck" / "step_00000007")
    assert CheckpointManager.validate(path) == []
    merged = CheckpointManager.load_tensors(path)
    assert set(merged) == set(full)
    for k, v in full.items():
        assert torch.equal(merged[k], v), k
    # ... into 4 tensor-parallel ranks, and into the unsharded model
    for r in range(4):
        fresh = ParallelEflaLM(m, "cpu", tp=SimpleNamespace(rank=r, world=4), seed=3)
        other = ParallelEflaLM(m, "cpu", tp=SimpleNamespace(rank=r, world=4), seed=99)
        other.load_reference_state(merged)
        for (n, a), (_, b) in zip(fresh.named_parameters(), other.named_parameters()):
            assert torch.equal(a, b), (r, n)
    single = EflaLM(m, "cpu", dtype=torch.bfloat16, seed=99)
    single.load_reference_state(merged)
    assert all(torch.equal(v, full[k]) for k, v in single.state_dict_reference().items())
    CheckpointManager.convert(path, tmp_path / "m.safetensors", "safetensors")
