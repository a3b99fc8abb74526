"""Byte-level BPE tokenizer: train / encode / decode / save / load / encode_file.

Same vocabulary construction as the reference (src/data/tokenizer.zig:58-214): ids 0..255
are the raw bytes, then ``<pad> <unk> <bos> <eos>``, then one id per learned merge, merges
chosen greedily by pair frequency over whitespace-delimited words and applied in learned
order when encoding (tokenizer.zig:336-361).  Unlike the reference, whose decoder
concatenates words and so loses the whitespace (tokenizer.zig:364-380), every word keeps
its leading whitespace as part of the piece, which makes ``decode(encode(s)) == s``.

File format (tokenizer.zig:272-288): ``u32 magic, u32 vocab``; per token ``u32 len, bytes``;
``u32 n_merges``; per merge ``u32 first, second, result``.  ``encode_file`` output
(tokenizer.zig:399-403): ``u64 n`` then u32 tokens.  Only BPE is implemented, as in the
reference (``unigram`` and ``word`` are named but absent there: tokenizer.zig:3-7, 45).
"""
from __future__ import annotations

import re
import struct
from collections import Counter

import numpy as np

from ..utils.formats import MAGIC_TOKENIZER, FormatError

SPECIAL_TOKENS = ("<pad>", "<unk>", "<bos>", "<eos>")
_PIECE = re.compile(rb"\s*\S+|\s+")


class Tokenizer:
    def __init__(self):
        self.vocab: list[bytes] = [bytes([b]) for b in range(256)] + \
            [s.encode() for s in SPECIAL_TOKENS]
        self.merges: list[tuple[int, int, int]] = []
        self._rank: dict[tuple[int, int], tuple[int, int]] = {}
        self.special = {s: 256 + i for i, s in enumerate(SPECIAL_TOKENS)}

    # ------------------------------------------------------------------------- training
    @classmethod
    def train_from_text(cls, text: str | bytes, vocab_size: int) -> "Tokenizer":
        self = cls()
        data = text.encode() if isinstance(text, str) else bytes(text)
        words = Counter(m.group(0) for m in _PIECE.finditer(data))
        seqs = {w: list(w) for w in words}
        n_merges = max(0, vocab_size - len(self.vocab))
        for _ in range(n_merges):
            pairs: Counter = Counter()
            for w, seq in seqs.items():
                f = words[w]
                for a, b in zip(seq, seq[1:]):
                    pairs[(a, b)] += f
            if not pairs:
                break
            # most frequent pair; ties broken by the smaller ids so training is deterministic
            (a, b), cnt = min(pairs.items(), key=lambda kv: (-kv[1], kv[0]))
            if cnt < 1:
                break
            new_id = len(self.vocab)
            self.vocab.append(self.vocab[a] + self.vocab[b])
            self.merges.append((a, b, new_id))
            for w, seq in seqs.items():
                if len(seq) < 2:
                    continue
                out, i = [], 0
                while i < len(seq):
                    if i + 1 < len(seq) and seq[i] == a and seq[i + 1] == b:
                        out.append(new_id)
                        i += 2
                    else:
                        out.append(seq[i])
                        i += 1
                seqs[w] = out
        self._index()
        return self

    @classmethod
    def train(cls, corpus_path, vocab_size: int) -> "Tokenizer":
        with open(corpus_path, "rb") as f:
            return cls.train_from_text(f.read(), vocab_size)

    def _index(self):
        self._rank = {(a, b): (i, r) for i, (a, b, r) in enumerate(self.merges)}
        self._cache: dict[bytes, list[int]] = {}

    # --------------------------------------------------------------------- encode / decode
    def _encode_piece(self, piece: bytes) -> list[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        seq = list(piece)
        while len(seq) > 1:
            best, best_i = None, -1
            for i, pr in enumerate(zip(seq, seq[1:])):
                r = self._rank.get(pr)
                if r is not None and (best is None or r[0] < best[0]):
                    best, best_i = r, i
            if best is None:
                break
            a, b = seq[best_i], seq[best_i + 1]
            out, i = [], 0
            while i < len(seq):  # merge every occurrence of the earliest-learned pair
                if i + 1 < len(seq) and seq[i] == a and seq[i + 1] == b:
                    out.append(best[1])
                    i += 2
                else:
                    out.append(seq[i])
                    i += 1
            seq = out
        if len(self._cache) < 200000:
            self._cache[piece] = seq
        return seq

    def encode(self, text: str | bytes, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        if isinstance(text, str) and text in self.special:  # tokenizer.zig:318-322
            return [self.special[text]]
        data = text.encode() if isinstance(text, str) else bytes(text)
        out = [self.special["<bos>"]] if add_bos else []
        for m in _PIECE.finditer(data):
            out.extend(self._encode_piece(m.group(0)))
        if add_eos:
            out.append(self.special["<eos>"])
        return out

    def decode_bytes(self, tokens) -> bytes:
        parts = []
        for t in tokens:
            t = int(t)
            if t < 0 or t >= len(self.vocab):
                raise ValueError(f"invalid token id {t}")
            if 256 <= t < 256 + len(SPECIAL_TOKENS):
                continue
            parts.append(self.vocab[t])
        return b"".join(parts)

    def decode(self, tokens) -> str:
        return self.decode_bytes(tokens).decode("utf-8", errors="replace")

    def vocab_size(self) -> int:
        return len(self.vocab)

    def token_id(self, token: str | bytes):
        b = token.encode() if isinstance(token, str) else token
        try:
            return self.vocab.index(b)
        except ValueError:
            return None

    def token(self, idx: int):
        return self.vocab[idx] if 0 <= idx < len(self.vocab) else None

    # ------------------------------------------------------------------------------- I/O
    def save(self, path) -> None:
        with open(path, "wb") as f:
            f.write(struct.pack("<II", MAGIC_TOKENIZER, len(self.vocab)))
            for tok in self.vocab:
                f.write(struct.pack("<I", len(tok)) + tok)
            f.write(struct.pack("<I", len(self.merges)))
            for a, b, r in self.merges:
                f.write(struct.pack("<III", a, b, r))

    @classmethod
    def load(cls, path) -> "Tokenizer":
        self = cls()
        with open(path, "rb") as f:
            hdr = f.read(8)
            if len(hdr) < 8:
                raise FormatError("truncated tokenizer file")
            mg, n = struct.unpack("<II", hdr)
            if mg != MAGIC_TOKENIZER:
                raise FormatError(f"bad tokenizer magic 0x{mg:08X}")
            vocab = []
            for _ in range(n):
                (ln,) = struct.unpack("<I", f.read(4))
                vocab.append(f.read(ln))
            (nm,) = struct.unpack("<I", f.read(4))
            merges = [struct.unpack("<III", f.read(12)) for _ in range(nm)]
        self.vocab, self.merges = vocab, [tuple(m) for m in merges]
        self._index()
        return self

    def encode_file(self, input_path, output_path) -> int:
        with open(input_path, "rb") as f:
            toks = self.encode(f.read())
        with open(output_path, "wb") as f:
            f.write(struct.pack("<Q", len(toks)))
            f.write(np.asarray(toks, dtype="<u4").tobytes())
        return len(toks)


def read_token_file(path) -> np.ndarray:
    """Reads an ``encode_file`` output back."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return np.frombuffer(f.read(4 * n), dtype="<u4")
