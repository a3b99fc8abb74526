"""Binary token datasets, shard writer/builder, data loader and sequence packing.

Counterparts of the reference's ``BinaryDataset`` (header + mmap of u32 tokens,
src/data/dataset.zig:14-107), ``ShardWriter`` (64-byte placeholder header, u32 LE tokens,
SHA-256: dataset.zig:110-159), ``DatasetBuilder`` (``shard_%06d.bin`` + ``.index``:
dataset.zig:162-285), ``DataLoader`` (non-overlapping windows of ``seq_len`` needing
``seq_len+1`` tokens, shuffle, ``drop_last``: dataset.zig:288-389), ``Batch`` and
``PackedSequence`` / ``packSequences`` (greedy first-fit that skips sequences that do not
fit: dataset.zig:405-465).  The reference computes the token offset from a rough estimate of
the shard-table size (dataset.zig:99-103); here the exact end of the header is used.

Additions: data-parallel striding by rank, a resumable cursor (epoch, position, RNG seed),
pinned host batches and a background prefetch thread.
"""
from __future__ import annotations

import hashlib
import os
import queue
import struct
import threading
from dataclasses import dataclass, field

import numpy as np
import torch

from ..utils import formats


class BinaryDataset:
    def __init__(self, path):
        self.path = str(path)
        with open(self.path, "rb") as f:
            self.num_tokens, self.shards, self.data_start = formats.read_dataset_header(f)
        size = os.path.getsize(self.path)
        avail = (size - self.data_start) // 4
        if avail < self.num_tokens:
            raise formats.FormatError(
                f"{self.path}: header promises {self.num_tokens} tokens, file holds {avail}")
        self.tokens = np.memmap(self.path, dtype="<u4", mode="r", offset=self.data_start,
                                shape=(self.num_tokens,))

    @classmethod
    def open(cls, path) -> "BinaryDataset":
        return cls(path)

    def get_tokens(self, start: int, count: int) -> np.ndarray:
        if start < 0 or start + count > self.num_tokens:
            raise IndexError(f"token range [{start}, {start + count}) outside the dataset")
        return self.tokens[start:start + count]

    def __len__(self):
        return self.num_tokens


def write_dataset(path, tokens, shards=None) -> None:
    """Single-file dataset: header + all tokens."""
    arr = np.asarray(tokens, dtype="<u4")
    with open(path, "wb") as f:
        formats.write_dataset_header(f, int(arr.size), shards or [])
        f.write(arr.tobytes())


class ShardWriter:
    def __init__(self, path):
        self.path = str(path)
        self.f = open(self.path, "wb")
        self.f.write(b"\0" * formats.SHARD_HEADER_BYTES)
        self.hash = hashlib.sha256()
        self.count = 0

    def write(self, tokens) -> None:
        b = np.asarray(tokens, dtype="<u4").tobytes()
        self.f.write(b)
        self.hash.update(b)
        self.count += len(b) // 4

    def close(self) -> formats.ShardInfo:
        self.f.close()
        return formats.ShardInfo(os.path.basename(self.path), self.count, self.hash.digest())


def read_shard(path) -> np.ndarray:
    return np.fromfile(path, dtype="<u4", offset=formats.SHARD_HEADER_BYTES)


class DatasetBuilder:
    """Streams tokens into ``shard_%06d.bin`` files of at most ``shard_tokens`` tokens and
    writes ``<name>.index`` (the dataset header with the shard table, no token data)."""

    def __init__(self, out_dir, shard_tokens: int = 1 << 24, name: str = "dataset"):
        self.dir, self.shard_tokens, self.name = str(out_dir), shard_tokens, name
        os.makedirs(self.dir, exist_ok=True)
        self.shards: list[formats.ShardInfo] = []
        self._w = None
        self.total = 0

    def add(self, tokens) -> None:
        arr = np.asarray(tokens, dtype="<u4")
        pos = 0
        while pos < arr.size:
            if self._w is None:
                self._w = ShardWriter(os.path.join(self.dir, f"shard_{len(self.shards):06d}.bin"))
            take = min(arr.size - pos, self.shard_tokens - self._w.count)
            self._w.write(arr[pos:pos + take])
            pos += take
            self.total += take
            if self._w.count >= self.shard_tokens:
                self.shards.append(self._w.close())
                self._w = None

    def finish(self) -> str:
        if self._w is not None:
            self.shards.append(self._w.close())
            self._w = None
        idx = os.path.join(self.dir, self.name + ".index")
        with open(idx, "wb") as f:
            formats.write_dataset_header(f, self.total, self.shards)
        return idx

    def merge(self, out_path) -> None:
        """Concatenates the shards into one single-file dataset."""
        with open(out_path, "wb") as f:
            formats.write_dataset_header(f, self.total, self.shards)
            for s in self.shards:
                f.write(read_shard(os.path.join(self.dir, s.path)).tobytes())


@dataclass
class Batch:
    input: torch.Tensor   # (B, T) int64
    target: torch.Tensor  # (B, T) int64


class DataLoader:
    """Windows ``[i*seq_len, i*seq_len + seq_len + 1)`` of the token stream; window i goes to
    data-parallel rank ``i % dp_world``.  ``state_dict`` / ``load_state_dict`` resume exactly."""

    def __init__(self, dataset, seq_len: int, batch_size: int, shuffle: bool = True,
                 drop_last: bool = True, seed: int = 0, dp_rank: int = 0, dp_world: int = 1,
                 pin: bool = False):
        self.ds, self.seq_len, self.batch_size = dataset, seq_len, batch_size
        self.shuffle, self.drop_last, self.seed = shuffle, drop_last, seed
        self.dp_rank, self.dp_world = dp_rank, dp_world
        self.pin = pin and torch.cuda.is_available()
        n_tok = len(dataset)
        self.num_windows = max(0, (n_tok - 1) // seq_len)
        self.epoch = 0
        self.pos = 0
        self._order = None
        self._build_order()

    def _build_order(self):
        idx = np.arange(self.num_windows, dtype=np.int64)
        if self.shuffle:
            np.random.default_rng([self.seed, self.epoch]).shuffle(idx)
        self._order = idx[self.dp_rank::self.dp_world]

    def __len__(self):
        n = len(self._order)
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    def reset(self):
        self.epoch += 1
        self.pos = 0
        self._build_order()

    def next(self):
        """Next ``Batch`` or None at the end of the epoch (call ``reset`` to start the next)."""
        n = len(self._order)
        if self.pos >= n or (self.drop_last and self.pos + self.batch_size > n):
            return None
        take = self._order[self.pos:self.pos + self.batch_size]
        self.pos += len(take)
        buf = np.empty((len(take), self.seq_len + 1), dtype=np.int64)
        for j, w in enumerate(take):
            buf[j] = self.ds.get_tokens(int(w) * self.seq_len, self.seq_len + 1)
        t = torch.from_numpy(buf)
        inp, tgt = t[:, :-1].contiguous(), t[:, 1:].contiguous()
        if self.pin:
            inp, tgt = inp.pin_memory(), tgt.pin_memory()
        return Batch(inp, tgt)

    def __iter__(self):
        while True:
            b = self.next()
            if b is None:
                return
            yield b

    def state_dict(self):
        return {"epoch": self.epoch, "pos": self.pos, "seed": self.seed}

    def load_state_dict(self, d):
        self.seed, self.epoch = int(d["seed"]), int(d["epoch"])
        self._build_order()
        self.pos = int(d["pos"])


class Prefetcher:
    """Runs ``loader.next()`` on a background thread, ``depth`` batches ahead
    (``data.prefetch_factor``).  An exception in the loader is re-raised by ``next``."""

    def __init__(self, loader: DataLoader, depth: int = 2):
        self.loader = loader
        self._consumed = loader.state_dict()
        self.q: queue.Queue = queue.Queue(maxsize=max(1, depth))
        self._stop = False
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()

    def _run(self):
        try:
            while not self._stop:
                b = self.loader.next()
                # the loader's cursor right after this batch travels with it, so a checkpoint
                # records what has been CONSUMED, not how far the thread has read ahead
                self.q.put((b, self.loader.state_dict()))
                if b is None:
                    return
        except BaseException as e:  # noqa: BLE001
            self.q.put(e)

    def next(self):
        item = self.q.get()
        if isinstance(item, BaseException):
            raise item
        b, self._consumed = item
        return b

    def state_dict(self):
        """The loader state after the last batch ``next`` handed out."""
        return getattr(self, "_consumed", None) or self.loader.state_dict()

    def close(self):
        self._stop = True
        try:
            while True:
                self.q.get_nowait()
        except queue.Empty:
            pass


@dataclass
class PackedSequence:
    tokens: np.ndarray                      # (max_len,) int64, zero padded
    sequence_ids: np.ndarray                # (max_len,) int32, -1 on padding
    cumulative_lengths: list[int] = field(default_factory=list)  # boundaries, starts with 0
    length: int = 0


def pack_sequences(sequences, max_len: int, align: int = 1) -> list[PackedSequence]:
    """Greedy packing in input order; a sequence longer than ``max_len`` is skipped, a
    sequence that does not fit the open pack closes it (dataset.zig:420-465).

    ``align`` > 1 starts every sequence on a multiple of ``align`` tokens (the gap is padding
    with sequence id -1), which is what the chunked EFLA kernels need to reset the recurrent
    state at document boundaries (``align=64``; see ``packed_batch``)."""
    packs, cur = [], None

    def new():
        return PackedSequence(np.zeros(max_len, np.int64), np.full(max_len, -1, np.int32), [0], 0)
    for seq in sequences:
        seq = np.asarray(seq, dtype=np.int64)
        if seq.size == 0 or seq.size > max_len:
            continue
        start = 0 if cur is None else -(-cur.length // align) * align
        if cur is None or start + seq.size > max_len:
            if cur is not None:
                packs.append(cur)
            cur, start = new(), 0
        sid = len(cur.cumulative_lengths) - 1
        cur.tokens[start:start + seq.size] = seq
        cur.sequence_ids[start:start + seq.size] = sid
        cur.length = start + seq.size
        cur.cumulative_lengths.append(cur.length)
    if cur is not None and cur.length:
        packs.append(cur)
    return packs


def packed_batch(packs, chunk: int = 64, pad_id: int = 0, ignore_index: int = -100):
    """Model inputs for packs made with ``pack_sequences(..., align=chunk)``: ``tokens`` and
    ``targets`` (B, L-1 rounded down to a multiple of ``chunk``; next-token targets,
    ``ignore_index`` on padding and on each document's last token) and ``resets``
    (B, T/chunk), set where a chunk starts a new document."""
    import torch
    L = len(packs[0].tokens)
    T = ((L - 1) // chunk) * chunk
    B = len(packs)
    tokens = np.full((B, T), pad_id, np.int64)
    targets = np.full((B, T), ignore_index, np.int64)
    resets = np.zeros((B, T // chunk), bool)
    for b, p in enumerate(packs):
        ids = p.sequence_ids
        tokens[b] = np.where(ids[:T] >= 0, p.tokens[:T], pad_id)
        same = (ids[:T] >= 0) & (ids[1:T + 1] == ids[:T])
        targets[b] = np.where(same, p.tokens[1:T + 1], ignore_index)
        starts = np.arange(0, T, chunk)
        prev = np.concatenate([[-2], ids[starts[1:] - 1]])
        resets[b] = (ids[starts] >= 0) & (ids[starts] != prev)
    return torch.from_numpy(tokens), torch.from_numpy(targets), torch.from_numpy(resets)
