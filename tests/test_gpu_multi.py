"""Multi-GPU tests: child processes under torchrun, one per GPU (skipped with < 2 GPUs).
NVLS is switched off in NCCL for these runs and the kernels under test use plain peer loads
and stores."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(what, nproc, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port",
           str(_free_port()), os.path.join(HERE, "multi_worker.py"), what]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _nranks():
    """All visible GPUs, rounded down to 2, 4 or 8."""
    n = _ngpu()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_zero_step_matches_nccl():
    out = _run("fused_vs_nccl", _nranks())
    assert "OK fused_vs_nccl" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_ag_gemm_and_gemm_rs():
    out = _run("tp_fused", _nranks())
    assert "OK tp_fused" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_context_parallel_efla_matches_single_gpu():
    out = _run("cp", _nranks())
    assert "OK cp" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_zero_stages_match_library_composition():
    out = _run("zero_stages", _nranks())
    assert "OK zero_stages" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("what", ["tp_model", "cp_model"])
def test_parallel_model_matches_single_gpu(what):
    # tensor parallel over at most 4 ranks (the model has 4 heads), context parallel over all
    n = min(4, _nranks()) if what == "tp_model" else _nranks()
    out = _run(what, n)
    assert f"OK {what}" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pipeline_stages_match_whole_model():
    out = _run("pipeline", 2)
    assert "OK pipeline" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_trainer_on_tensor_parallel_mesh_and_sharded_checkpoint():
    out = _run("train_tp", 2)
    assert "OK train_tp" in out
