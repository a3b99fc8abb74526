"""Modal launcher (counterpart of the reference's cloud/modal/train.py:64-377): an app
``efla-trainer`` with ``train / evaluate / generate / status`` on ``B200:8``, a one-GPU
``smoke_test``, volumes at ``/data`` and ``/checkpoints``, upload / download helpers for
those volumes, and a local entry point ``main(action=...)``.  Each action shells out to the CLI (``python -m ceo_b200.cli``), under
``torchrun`` for the multi-GPU ones.  ``modal`` is imported lazily so the module can be
imported (and its command lines tested) on machines without it.
"""
from __future__ import annotations

import os
import subprocess
import sys

APP_NAME = "efla-trainer"
REMOTE_ROOT = "/workspace/ceo_b200"   # where the image holds this repository
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
             .pip_install("torch", "numpy").add_local_dir(".", REMOTE_ROOT))
    app = modal.App(APP_NAME, image=image)
    data = modal.Volume.from_name("efla-data", create_if_missing=True)
    ckpt = modal.Volume.from_name("efla-checkpoints", create_if_missing=True)
    vols = {DATA_DIR: data, CKPT_DIR: ckpt}

    @app.function(gpu=GPU_TRAIN, volumes=vols, timeout=24 * 3600, retries=0)
    def train(config: str = "configs/efla_1p3b.yaml", resume: str = ""):
        os.chdir(REMOTE_ROOT)
        subprocess.check_call([sys.executable, "-m", "ceo_b200.build"])
        return run_action("train", config=config, resume=resume or None)

    @app.function(gpu=GPU_SMOKE, volumes=vols, timeout=1800)
    def smoke_test():
        os.chdir(REMOTE_ROOT)
        subprocess.check_call([sys.executable, "-m", "ceo_b200.build"])
        return run_action("smoke_test")

    @app.function(gpu=GPU_SMOKE, volumes=vols, timeout=3600)
    def evaluate(checkpoint: str, data: str):
        os.chdir(REMOTE_ROOT)
        return run_action("evaluate", checkpoint=checkpoint, data=data)

    @app.function(gpu=GPU_SMOKE, volumes=vols, timeout=3600)
    def generate(checkpoint: str, prompt: str = "", max_tokens: int = 64):
        os.chdir(REMOTE_ROOT)
        return run_action("generate", checkpoint=checkpoint, prompt=prompt, max_tokens=max_tokens)

    @app.function(volumes=vols)
    def status():
        return run_action("status")

    return app


# ---- volume transfers -------------------------------------------------------------------
# Counterparts of the reference's upload / download helpers and the four transfer actions of
# its local entry point (cloud/modal/train.py:251-302, 344-377).  They talk to anything with
# Modal's volume interface (``batch_upload()`` -> put_file / put_directory, ``read_file(path)``
# -> byte chunks, ``listdir(path, recursive=True)`` -> entries with ``path`` and ``type``),
# which lets the tests drive them with an in-memory stand-in.
VOLUME_NAMES = {"data": "efla-data", "checkpoint": "efla-checkpoints"}
TRANSFER_ACTIONS = {"upload-data": ("data", "up"), "upload-checkpoint": ("checkpoint", "up"),
                    "download-data-file": ("data", "file"),
                    "download-checkpoint": ("checkpoint", "tree")}


def _remote(path: str) -> str:
    clean = (path or "").strip("/")
    if not clean:
        raise ValueError("the remote path must not be empty")
    return clean


def volume_upload(volume, local_source: str, remote_path: str, force: bool = False) -> str:
    """Copies a local file or directory tree into the volume; returns the remote path used."""
    src = os.path.abspath(os.path.expanduser(local_source))
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    dst = _remote(remote_path)
    with volume.batch_upload(force=force) as batch:
        (batch.put_directory if os.path.isdir(src) else batch.put_file)(src, dst)
    return dst


def volume_download_file(volume, remote_path: str, local_path: str) -> int:
    """One file out of the volume; returns the number of bytes written."""
    dst = os.path.abspath(os.path.expanduser(local_path))
    os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
    n = 0
    with open(dst, "wb") as f:
        for chunk in volume.read_file(_remote(remote_path)):
            f.write(chunk)
            n += len(chunk)
    return n


def _entry(e):
    """(path, is_directory) of a volume listing entry (object or plain string)."""
    path = getattr(e, "path", e if isinstance(e, str) else "")
    kind = getattr(e, "type", None)
    is_dir = "dir" in str(getattr(kind, "name", kind)).lower() if kind is not None \
        else str(path).endswith("/")
    return str(path).strip("/"), is_dir


def volume_download_tree(volume, remote_path: str, local_path: str) -> list[str]:
    """A directory of the volume (a checkpoint, say) into ``local_path``; returns the files
    written, relative to it.  Raises FileNotFoundError when nothing is there."""
    root = _remote(remote_path)
    out_root = os.path.abspath(os.path.expanduser(local_path))
    os.makedirs(out_root, exist_ok=True)
    written = []
    for e in volume.listdir(root, recursive=True):
        path, is_dir = _entry(e)
        if not path or not (path == root or path.startswith(root + "/")):
            continue
        rel = os.path.relpath(path, root)
        target = os.path.join(out_root, rel)
        if is_dir:
            os.makedirs(target, exist_ok=True)
            continue
        volume_download_file(volume, path, target)
        written.append(rel)
    if not written:
        raise FileNotFoundError(root)
    return sorted(written)


def _volume(kind: str):
    import modal
    return modal.Volume.from_name(VOLUME_NAMES[kind], create_if_missing=True)


def transfer(action: str, local_path: str = "", remote_path: str = "", checkpoint: str = "",
             force: bool = False, volume=None):
    """The four transfer actions; ``volume`` overrides the named Modal volume (tests)."""
    kind, mode = TRANSFER_ACTIONS[action]
    vol = volume if volume is not None else _volume(kind)
    if mode == "up":
        if not local_path or not remote_path:
            raise ValueError(f"{action} needs local_path and remote_path")
        return volume_upload(vol, local_path, remote_path, force)
    if mode == "file":
        if not local_path or not remote_path:
            raise ValueError(f"{action} needs local_path and remote_path")
        return volume_download_file(vol, remote_path, local_path)
    if not local_path or not (checkpoint or remote_path):
        raise ValueError(f"{action} needs local_path and checkpoint")
    return volume_download_tree(vol, checkpoint or remote_path, local_path)


def main(action: str = "smoke_test", **kw) -> int:
    """Local entry point: train | evaluate | generate | status | smoke_test run the CLI;
    upload-data | upload-checkpoint | download-data-file | download-checkpoint move files
    between this machine and the volumes."""
    action = action.strip().lower()
    if action in TRANSFER_ACTIONS:
        transfer(action, **kw)
        return 0
    return run_action(action.replace("-", "_"), **kw)


if __name__ == "__main__":
    sys.exit(main(*(sys.argv[1:2] or ["smoke_test"])))
