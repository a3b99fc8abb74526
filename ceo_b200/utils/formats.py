"""Binary file formats shared with the reference: checkpoint tensor file, dataset file and
shards, tokenizer file.  All integers little-endian.

The reference writes its magic numbers as hex-speak that is not a valid literal
(``0xEFLACK01`` src/checkpoint/manager.zig:185, ``0xEFLAOP01`` manager.zig:244, ``0xEFLAD001``
src/data/dataset.zig:33, ``0xEFLA0001`` src/data/tokenizer.zig:237); the values here apply
the substitution L->1, K->C, O->0, P->9 and readers accept exactly these.

tensors.bin (manager.zig:184-230): ``u32 magic, u32 version=1, u32 n``; per tensor
``u32 name_len, name, u32 ndim, u64 dims[ndim], u8 dtype, u64 offset, u64 size,
u8 sha256[32]``; then the raw tensor bytes in index order (offsets are relative to the start
of the data section).  The reference stores the digest of the empty string as a placeholder
(manager.zig:215-217); this writer stores the real SHA-256 of each tensor's bytes and the
reader verifies it unless the placeholder is found.
"""
from __future__ import annotations

import hashlib
import io
import struct
from dataclasses import dataclass

import numpy as np
import torch

MAGIC_CHECKPOINT = 0xEF1ACC01
MAGIC_OPTIMIZER = 0xEF1A0901
MAGIC_DATASET = 0xEF1AD001
MAGIC_TOKENIZER = 0xEF1A0001
VERSION = 1
EMPTY_SHA256 = hashlib.sha256(b"").digest()

# DType enum values of the reference (src/tensor/dtype.zig:3-13)
DTYPE_CODES = {"fp32": 0, "fp16": 1, "bf16": 2, "fp8_e4m3": 3, "fp8_e5m2": 4, "fp4": 5,
               "int8": 6, "int32": 7, "int64": 8, "bool": 9}
_TORCH_TO_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2,
                  torch.float8_e4m3fn: 3, torch.float8_e5m2: 4, torch.int8: 6, torch.int32: 7,
                  torch.int64: 8, torch.bool: 9}
_CODE_TO_TORCH = {v: k for k, v in _TORCH_TO_CODE.items()}
_ITEMSIZE = {0: 4, 1: 2, 2: 2, 3: 1, 4: 1, 6: 1, 7: 4, 8: 8, 9: 1}


class FormatError(ValueError):
    pass


def tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


def bytes_to_tensor(buf: bytes, code: int, dims) -> torch.Tensor:
    dt = _CODE_TO_TORCH.get(code)
    if dt is None:
        raise FormatError(f"unsupported dtype code {code}")
    raw = torch.frombuffer(bytearray(buf), dtype=torch.uint8)
    return raw.view(dt).reshape(tuple(dims)).clone()


@dataclass
class TensorEntry:
    name: str
    dims: tuple
    dtype_code: int
    offset: int
    size: int
    sha256: bytes


def write_tensor_file(path, tensors: dict, magic: int = MAGIC_CHECKPOINT) -> list[TensorEntry]:
    """``tensors``: ordered name -> torch.Tensor.  Returns the index entries written."""
    entries, blobs, off = [], [], 0
    for name, t in tensors.items():
        code = _TORCH_TO_CODE.get(t.dtype)
        if code is None:
            raise FormatError(f"{name}: dtype {t.dtype} has no code in the checkpoint format")
        b = tensor_bytes(t)
        entries.append(TensorEntry(name, tuple(t.shape), code, off, len(b),
                                   hashlib.sha256(b).digest()))
        blobs.append(b)
        off += len(b)
    with open(path, "wb") as f:
        f.write(struct.pack("<III", magic, VERSION, len(entries)))
        for e in entries:
            nb = e.name.encode()
            f.write(struct.pack("<I", len(nb)) + nb)
            f.write(struct.pack("<I", len(e.dims)))
            f.write(struct.pack(f"<{len(e.dims)}Q", *e.dims))
            f.write(struct.pack("<BQQ", e.dtype_code, e.offset, e.size))
            f.write(e.sha256)
        for b in blobs:
            f.write(b)
    return entries


def read_tensor_index(f, magic: int = MAGIC_CHECKPOINT):
    """Reads the header + index from an open binary file; returns (entries, data_start)."""
    hdr = f.read(12)
    if len(hdr) < 12:
        raise FormatError("truncated tensor file")
    mg, ver, n = struct.unpack("<III", hdr)
    if mg != magic:
        raise FormatError(f"bad magic 0x{mg:08X} (expected 0x{magic:08X})")
    if ver != VERSION:
        raise FormatError(f"unsupported version {ver}")
    entries = []
    for _ in range(n):
        (nl,) = struct.unpack("<I", f.read(4))
        name = f.read(nl).decode()
        (nd,) = struct.unpack("<I", f.read(4))
        if nd > 8:
            raise FormatError(f"{name}: {nd} dimensions")
        dims = struct.unpack(f"<{nd}Q", f.read(8 * nd)) if nd else ()
        code, off, size = struct.unpack("<BQQ", f.read(17))
        sha = f.read(32)
        entries.append(TensorEntry(name, tuple(dims), code, off, size, sha))
    return entries, f.tell()


def read_tensor_file(path, magic: int = MAGIC_CHECKPOINT, verify: bool = True,
                     names=None) -> dict:
    out = {}
    with open(path, "rb") as f:
        entries, start = read_tensor_index(f, magic)
        for e in entries:
            if names is not None and e.name not in names:
                continue
            f.seek(start + e.offset)
            b = f.read(e.size)
            if len(b) != e.size:
                raise FormatError(f"{e.name}: truncated data")
            if verify and e.sha256 != EMPTY_SHA256 and hashlib.sha256(b).digest() != e.sha256:
                raise FormatError(f"{e.name}: checksum mismatch (corrupted checkpoint)")
            expect = int(np.prod(e.dims, dtype=np.int64)) * _ITEMSIZE.get(e.dtype_code, 0) \
                if e.dims else _ITEMSIZE.get(e.dtype_code, 0)
            if expect != e.size:
                raise FormatError(f"{e.name}: size {e.size} does not match shape {e.dims}")
            out[e.name] = bytes_to_tensor(b, e.dtype_code, e.dims)
    return out


# ------------------------------------------------------------------------------- dataset
@dataclass
class ShardInfo:
    path: str
    num_tokens: int
    sha256: bytes


def write_dataset_header(f, num_tokens: int, shards: list[ShardInfo]):
    """dataset.zig:28-58 / 269-281: magic, version, u64 num_tokens, u32 num_shards, per shard
    (u32 path_len, path, u64 tokens, sha256[32]); u32 LE tokens follow."""
    f.write(struct.pack("<IIQI", MAGIC_DATASET, VERSION, num_tokens, len(shards)))
    for s in shards:
        pb = s.path.encode()
        f.write(struct.pack("<I", len(pb)) + pb)
        f.write(struct.pack("<Q", s.num_tokens))
        f.write(s.sha256)


def read_dataset_header(f):
    hdr = f.read(20)
    if len(hdr) < 20:
        raise FormatError("truncated dataset header")
    mg, ver, ntok, nsh = struct.unpack("<IIQI", hdr)
    if mg != MAGIC_DATASET:
        raise FormatError(f"bad dataset magic 0x{mg:08X}")
    if ver != VERSION:
        raise FormatError(f"unsupported dataset version {ver}")
    shards = []
    for _ in range(nsh):
        (pl,) = struct.unpack("<I", f.read(4))
        path = f.read(pl).decode()
        (st,) = struct.unpack("<Q", f.read(8))
        shards.append(ShardInfo(path, st, f.read(32)))
    return ntok, shards, f.tell()


SHARD_HEADER_BYTES = 64  # zero-filled placeholder header of a shard file (dataset.zig:129-140)
