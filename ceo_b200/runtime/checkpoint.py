"""Checkpoint manager: ``{dir}/step_{step:08d}/`` with ``metadata.json``, ``tensors.bin``,
``optimizer.bin`` / ``optimizer.rank{r}.bin``, ``rng.bin`` and ``config.yaml``.

Directory layout, metadata fields and the tensor-file format are the reference's
(src/checkpoint/manager.zig:67-246; formats in ``utils/formats.py``); ``evaluate`` and
``generate`` expect ``{ckpt}/config.yaml`` (src/main.zig:185,232), which the reference never
writes and this manager does.  Where the reference stops short this one goes on: the reader
works (the reference seeks to a relative offset as if absolute: manager.zig:372-375), real
per-tensor SHA-256, optimizer state (fp32 master + moments, one file per rank so a sharded
run writes in parallel), RNG, loader cursor and scheduler step, retention of the newest
``keep_last_n`` directories (manager.zig:382-423), asynchronous save from a host snapshot
(``checkpoint.async_save``), ``convert`` to safetensors / torch, and re-sharding of the
optimizer state when the world size or the ownership layout changes between save and load.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import struct
import threading
import time

import torch

from ..utils import formats

_STEP_RE = re.compile(r"^step_(\d{8})$")


def parse_step(name: str):
    m = _STEP_RE.match(name)
    return int(m.group(1)) if m else None


class CheckpointManager:
    def __init__(self, directory, keep_last_n: int = 5, save_optimizer: bool = True,
                 async_save: bool = False, rank: int = 0, world: int = 1):
        self.dir = str(directory)
        self.keep_last_n, self.save_optimizer = keep_last_n, save_optimizer
        self.async_save, self.rank, self.world = async_save, rank, world
        self._thread = None
        self._error = None

    # ------------------------------------------------------------------------- listing
    def path_for(self, step: int) -> str:
        return os.path.join(self.dir, f"step_{step:08d}")

    def list_checkpoints(self) -> list[int]:
        if not os.path.isdir(self.dir):
            return []
        steps = [parse_step(n) for n in os.listdir(self.dir)]
        return sorted(s for s in steps if s is not None
                      and os.path.exists(os.path.join(self.path_for(s), "metadata.json")))

    def latest(self):
        steps = self.list_checkpoints()
        return self.path_for(steps[-1]) if steps else None

    # --------------------------------------------------------------------------- save
    def save(self, step: int, tensors: dict, metadata: dict, optimizer_state: dict | None = None,
             rng_state: bytes | None = None, config_yaml: str | None = None,
             extra: dict | None = None, shard_timeout: float = 600.0,
             tensor_shards: dict | None = None, shard_rank: int = 0, shard_world: int = 1) -> str:
        """``tensors``: name -> tensor (reference names/orientation), written by rank 0.
        ``optimizer_state``: name -> tensor, this rank's slice, written by every rank.
        ``tensor_shards`` (tensor / pipeline parallelism): name -> (tensor, shard_dim or None),
        what model shard ``shard_rank`` of ``shard_world`` holds (shards ordered pipeline stage
        first, tensor-parallel rank second; a slice along ``shard_dim`` or a whole tensor).
        Each shard holder writes ``tensors.rank{shard_rank}.bin`` and rank 0 writes
        ``tensors.index.json``, from which ``load_tensors`` rebuilds the full tensors, so every
        reader sees one model whatever layout wrote it.  Pass it on the ranks that hold
        data-parallel replica 0 only.
        Every rank drops a ``rank{r}.done`` marker once its files are complete; rank 0 commits
        ``metadata.json`` (and prunes older checkpoints) only after all markers are there, so a
        directory that ``latest()`` returns always holds every shard."""
        self.wait()
        path = self.path_for(step)
        host_tensors = {k: v.detach().to("cpu", copy=True) for k, v in tensors.items()} \
            if self.rank == 0 else {}
        host_shards = None
        if tensor_shards is not None:
            # a slice is stored as "name@dim" (this file's slice of the full tensor along dim)
            host_shards = {(k if v[1] is None else f"{k}@{int(v[1])}"):
                           v[0].detach().to("cpu", copy=True) for k, v in tensor_shards.items()}
        host_opt = None
        if optimizer_state is not None and self.save_optimizer:
            host_opt = {k: v.detach().to("cpu", copy=True) for k, v in optimizer_state.items()}

        def work():
            try:
                os.makedirs(path, exist_ok=True)
                if host_opt is not None:
                    name = "optimizer.bin" if self.world == 1 else f"optimizer.rank{self.rank}.bin"
                    formats.write_tensor_file(os.path.join(path, name), host_opt,
                                              formats.MAGIC_OPTIMIZER)
                if host_shards is not None:
                    formats.write_tensor_file(os.path.join(path, f"tensors.rank{shard_rank}.bin"),
                                              host_shards)
                    if self.rank == 0:
                        with open(os.path.join(path, "tensors.index.json"), "w") as f:
                            json.dump({"files": [f"tensors.rank{r}.bin"
                                                 for r in range(shard_world)]}, f, indent=1)
                with open(os.path.join(path, f"rank{self.rank}.done"), "w") as f:
                    f.write(str(int(step)))
                if self.rank == 0:
                    if host_shards is None:
                        formats.write_tensor_file(os.path.join(path, "tensors.bin"), host_tensors)
                    if rng_state is not None:
                        with open(os.path.join(path, "rng.bin"), "wb") as f:
                            f.write(rng_state)
                    if config_yaml is not None:
                        with open(os.path.join(path, "config.yaml"), "w") as f:
                            f.write(config_yaml)
                    md = {"step": int(step), "epoch": 0, "tokens_seen": 0, "loss": 0.0,
                          "learning_rate": 0.0, "timestamp": int(time.time()),
                          "git_revision": "0" * 40, "config_hash": "0" * 64,
                          "world_size": self.world}
                    md.update(metadata)
                    md["has_optimizer"] = host_opt is not None
                    if extra:
                        md["extra"] = extra
                    deadline = time.time() + shard_timeout
                    missing = list(range(self.world))
                    while missing:
                        missing = [r for r in missing
                                   if not os.path.exists(os.path.join(path, f"rank{r}.done"))]
                        if missing and time.time() > deadline:
                            raise TimeoutError(f"checkpoint {path}: ranks {missing} never "
                                               "finished writing their shards")
                        if missing:
                            time.sleep(0.05)
                    tmp = os.path.join(path, "metadata.json.tmp")
                    with open(tmp, "w") as f:
                        json.dump(md, f, indent=1)
                    os.replace(tmp, os.path.join(path, "metadata.json"))  # commit point
                    self.cleanup_old()
            except BaseException as e:  # noqa: BLE001
                self._error = e

        if self.async_save:
            self._thread = threading.Thread(target=work, daemon=True)
            self._thread.start()
        else:
            work()
            self._raise()
        return path

    def wait(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        self._raise()

    def _raise(self):
        if self._error is not None:
            e, self._error = self._error, None
            raise e

    def cleanup_old(self):
        steps = self.list_checkpoints()
        if self.keep_last_n > 0:
            for s in steps[:-self.keep_last_n]:
                shutil.rmtree(self.path_for(s), ignore_errors=True)

    # --------------------------------------------------------------------------- load
    @staticmethod
    def read_metadata(path) -> dict:
        with open(os.path.join(path, "metadata.json")) as f:
            return json.load(f)

    @staticmethod
    def load_tensors(path, verify: bool = True) -> dict:
        """The model's full tensors under the reference's names: ``tensors.bin``, or, for a
        checkpoint written under tensor parallelism, the per-rank files merged through
        ``tensors.index.json`` (sharded tensors concatenated along their shard dimension)."""
        single = os.path.join(path, "tensors.bin")
        if os.path.exists(single):
            return formats.read_tensor_file(single, verify=verify)
        with open(os.path.join(path, "tensors.index.json")) as f:
            idx = json.load(f)
        whole, slices = {}, {}
        for n in idx["files"]:  # file order = (pipeline stage, tensor-parallel rank)
            for key, t in formats.read_tensor_file(os.path.join(path, n), verify=verify).items():
                if "@" in key:
                    name, dim = key.rsplit("@", 1)
                    slices.setdefault(name, (int(dim), []))[1].append(t)
                else:
                    whole.setdefault(key, t)
        for name, (dim, parts) in slices.items():
            whole[name] = torch.cat(parts, dim=dim)
        return whole

    def load_optimizer(self, path, flat=None) -> dict | None:
        """This rank's optimizer state.  Saved with the same world size and ownership layout:
        this rank's own file.  Otherwise (``flat``: the new run's ``FlatParams``) the flat-shard
        tensors (master weights, moments: everything as long as ``master``) are rebuilt from
        all ranks' files through the saved ownership map and re-split; replicated entries
        (``step_count``, ``side.*``) come from one file unchanged; ``muon.*`` entries are the
        union over all files (the caller keeps the matrices it now owns).
        Returns None when the checkpoint carries no optimizer state; raises
        ``CheckpointCorrupted`` when it says it does and a shard is missing."""
        from ..utils import errors
        md = self.read_metadata(path)
        saved_world = int(md.get("world_size", 1))
        saved_layout = (md.get("extra") or {}).get("flat_layout") or \
            {"layout": "contiguous", "world": saved_world}
        files = [os.path.join(path, "optimizer.bin")] if saved_world == 1 else \
            [os.path.join(path, f"optimizer.rank{r}.bin") for r in range(saved_world)]
        present = [os.path.exists(p) for p in files]
        if not any(present) and not md.get("has_optimizer", False):
            return None
        same = saved_world == self.world and (
            flat is None or saved_layout.get("layout", "contiguous") == flat.layout)
        if same:
            mine = files[0] if self.world == 1 else files[self.rank]
            if not os.path.exists(mine):
                raise errors.CheckpointCorrupted(f"{path}: optimizer shard of rank {self.rank} "
                                                 "is missing")
            return formats.read_tensor_file(mine, formats.MAGIC_OPTIMIZER)
        if not all(present):
            gone = [os.path.basename(p) for p, ok in zip(files, present) if not ok]
            raise errors.CheckpointCorrupted(f"{path}: optimizer shards missing: {gone}")
        if flat is None:
            raise ValueError("re-sharding optimizer state needs the new run's FlatParams")
        parts = [formats.read_tensor_file(p, formats.MAGIC_OPTIMIZER) for p in files]
        shard_len = parts[0]["master"].numel()
        out = {}
        for k, v in parts[0].items():
            if k.startswith(("muon.", "side.")) or k == "step_count":
                continue
            if v.numel() == shard_len and all(k in p for p in parts):
                out[k] = flat.reshard([p[k] for p in parts], saved_layout)
        for k, v in parts[0].items():
            if k == "step_count" or k.startswith("side."):
                out[k] = v
        for p in parts:
            for k, v in p.items():
                if k.startswith("muon."):
                    out.setdefault(k, v)
        return out

    @staticmethod
    def load_rng(path):
        p = os.path.join(path, "rng.bin")
        if not os.path.exists(p):
            return None
        with open(p, "rb") as f:
            return f.read()

    # ----------------------------------------------------------------- validate / convert
    @staticmethod
    def validate(path) -> list[str]:
        """Returns a list of problems (empty = valid): files present, index parses, sizes
        consistent, every checksum matches."""
        problems = []
        sharded = os.path.exists(os.path.join(path, "tensors.index.json"))
        for need in ("metadata.json", "tensors.index.json" if sharded else "tensors.bin"):
            if not os.path.exists(os.path.join(path, need)):
                problems.append(f"missing {need}")
        if problems:
            return problems
        try:
            md = json.load(open(os.path.join(path, "metadata.json")))
            if md.get("has_optimizer"):
                w = int(md.get("world_size", 1))
                names = ["optimizer.bin"] if w == 1 else [f"optimizer.rank{r}.bin" for r in range(w)]
                for n in names:
                    if not os.path.exists(os.path.join(path, n)):
                        problems.append(f"missing {n}")
        except Exception as e:  # noqa: BLE001
            problems.append(f"metadata.json: {e}")
        try:
            CheckpointManager.load_tensors(path, verify=True)
        except Exception as e:  # noqa: BLE001
            problems.append(f"{'tensors.rank*.bin' if sharded else 'tensors.bin'}: {e}")
        return problems

    @staticmethod
    def convert(input_path, output_path, fmt: str) -> None:
        """``efla_native`` (re-write), ``pytorch`` (torch.save of the dict) or ``safetensors``."""
        tensors = CheckpointManager.load_tensors(input_path) if os.path.isdir(input_path) \
            else formats.read_tensor_file(input_path)
        if fmt == "efla_native":
            formats.write_tensor_file(output_path, tensors)
        elif fmt == "pytorch":
            torch.save(tensors, output_path)
        elif fmt == "safetensors":
            write_safetensors(output_path, tensors)
        else:
            raise ValueError(f"unknown format {fmt!r} (efla_native | safetensors | pytorch)")


_ST_DTYPES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
              torch.int64: "I64", torch.int32: "I32", torch.int8: "I8", torch.bool: "BOOL",
              torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2"}


def write_safetensors(path, tensors: dict) -> None:
    """Minimal safetensors writer: u64 header length, JSON header, raw little-endian data."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        b = formats.tensor_bytes(t)
        header[name] = {"dtype": _ST_DTYPES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_safetensors(path) -> dict:
    inv = {v: k for k, v in _ST_DTYPES.items()}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        raw = torch.frombuffer(bytearray(data[a:b]), dtype=torch.uint8)
        out[name] = raw.view(inv[e["dtype"]]).reshape(e["shape"]).clone()
    return out
