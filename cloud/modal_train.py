"""Modal launcher (counterpart of the reference's cloud/modal/train.py:64-377): an app
``efla-trainer`` with ``train / evaluate / generate / status`` on ``B200:8``, a one-GPU
``smoke_test``, volumes at ``/data`` and ``/checkpoints``, and a local entry point
``main(action=...)``.  Each action shells out to the CLI (``python -m ceo_b200.cli``), under
``torchrun`` for the multi-GPU ones.  ``modal`` is imported lazily so the module can be
imported (and its command lines tested) on machines without it.
"""
from __future__ import annotations

import os
import subprocess
import sys

APP_NAME = "efla-trainer"
GPU_TRAIN = "B200:8"
GPU_SMOKE = "B200"
DATA_DIR = "/data"
CKPT_DIR = "/checkpoints"


def torchrun_prefix(n_gpus: int, port: int = 29500) -> list[str]:
    if n_gpus <= 1:
        return [sys.executable, "-m", "ceo_b200.cli"]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
            f"--nproc-per-node={n_gpus}", "--master-addr", "127.0.0.1", "--master-port",
            str(port), "-m", "ceo_b200.cli"]


def command_for(action: str, n_gpus: int = 8, **kw) -> list[str]:
    """The command line an action runs (pure function: used by the tests)."""
    if action == "train":
        cmd = torchrun_prefix(n_gpus) + ["train", "--config", kw.get("config", "configs/train.yaml"),
                                         "--checkpoint-dir", kw.get("checkpoint_dir", CKPT_DIR)]
        if kw.get("data"):
            cmd += ["--data", kw["data"]]
        if kw.get("resume"):
            cmd += ["--resume", kw["resume"]]
        return cmd
    if action == "evaluate":
        return torchrun_prefix(1) + ["evaluate", "--checkpoint", kw["checkpoint"], "--data",
                                     kw["data"]]
    if action == "generate":
        return torchrun_prefix(1) + ["generate", "--checkpoint", kw["checkpoint"], "--prompt",
                                     kw.get("prompt", ""), "--max-tokens",
                                     str(kw.get("max_tokens", 64))]
    if action == "smoke_test":
        return torchrun_prefix(1) + ["smoke-test"]
    if action == "status":
        return torchrun_prefix(1) + ["checkpoint", "list", "--dir", kw.get("checkpoint_dir", CKPT_DIR)]
    raise ValueError(f"unknown action {action!r}")


def run_action(action: str, **kw) -> int:
    env = dict(os.environ)
    env.setdefault("NCCL_DEBUG", "WARN")
    return subprocess.run(command_for(action, **kw), env=env).returncode


def build_app():
    """Creates the Modal app (needs the ``modal`` package)."""
    import modal

    image = (modal.Image.from_registry("nvidia/cuda:12.9.0-devel-ubuntu24.04", add_python="3.12")
             .pip_install("torch", "numpy").add_local_dir(".", "/root/repo"))
    app = modal.App(APP_NAME, image=image)
    data = modal.Volume.from_name("efla-data", create_if_missing=True)
    ckpt = modal.Volume.from_name("efla-checkpoints", create_if_missing=True)
    vols = {DATA_DIR: data, CKPT_DIR: ckpt}

    @app.function(gpu=GPU_TRAIN, volumes=vols, timeout=24 * 3600, retries=0)
    def train(config: str = "configs/efla_1p3b.yaml", resume: str = ""):
        os.chdir("/root/repo")
        subprocess.check_call([sys.executable, "-m", "ceo_b200.build"])
        return run_action("train", config=config, resume=resume or None)

    @app.function(gpu=GPU_SMOKE, volumes=vols, timeout=1800)
    def smoke_test():
        os.chdir("/root/repo")
        subprocess.check_call([sys.executable, "-m", "ceo_b200.build"])
        return run_action("smoke_test")

    @app.function(gpu=GPU_SMOKE, volumes=vols, timeout=3600)
    def evaluate(checkpoint: str, data: str):
        os.chdir("/root/repo")
        return run_action("evaluate", checkpoint=checkpoint, data=data)

    @app.function(gpu=GPU_SMOKE, volumes=vols, timeout=3600)
    def generate(checkpoint: str, prompt: str = "", max_tokens: int = 64):
        os.chdir("/root/repo")
        return run_action("generate", checkpoint=checkpoint, prompt=prompt, max_tokens=max_tokens)

    @app.function(volumes=vols)
    def status():
        return run_action("status")

    return app


def main(action: str = "smoke_test", **kw) -> int:
    return run_action(action, **kw)


if __name__ == "__main__":
    sys.exit(main(*(sys.argv[1:2] or ["smoke_test"])))
