"""Evaluation and generation.

Surface of the reference's evaluator (src/eval/evaluator.zig): ``Evaluator`` with
``evaluate_perplexity`` (58-102) and ``evaluate_long_context`` (113-128), ``Generator`` with
``generate`` (170-191), ``generate_greedy`` (194-210) and ``sample_top_p`` (213-259), and
``benchmark_throughput`` (263-308).  The reference builds a fresh random CPU model and ignores
the checkpoint (29-51), returns a constant loss (104-110), emits spaces instead of tokens
(170-191), samples top-p over the unsorted distribution (213-259) and times an empty loop
(287-297).  Here the checkpoint is loaded, the loss is the model's, generation is a
recurrent decode that carries one d x d state per head and layer (constant memory in the
context length), nucleus sampling sorts the probabilities, and the benchmark times real
steps with CUDA events.
"""
from __future__ import annotations

import math
import os
import time

import torch

from ..data.dataset import BinaryDataset, DataLoader
from ..models.model import EflaLM
from ..ops import nn as K
from ..utils.config import Config
from .checkpoint import CheckpointManager


def load_model(checkpoint_path: str | None, cfg: Config | None = None, device=None):
    """Builds the model from ``{ckpt}/config.yaml`` (or ``cfg``) and loads ``tensors.bin``."""
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if cfg is None:
        cfg = Config.parse_from_file(os.path.join(checkpoint_path, "config.yaml"))
    dev = torch.device(device)
    model = EflaLM(cfg.model, dev, dtype=torch.bfloat16 if dev.type == "cuda" else None,
                   seed=cfg.runtime.seed)
    if checkpoint_path:
        model.load_reference_state(CheckpointManager.load_tensors(checkpoint_path))
    model.eval()
    return model, cfg


class Evaluator:
    def __init__(self, model: EflaLM, cfg: Config):
        self.model, self.cfg = model, cfg
        self.device = model.embed_tokens.device

    @torch.no_grad()
    def evaluate_perplexity(self, data_path: str, max_tokens: int | None = None,
                            seq_len: int | None = None, batch_size: int = 1) -> dict:
        seq_len = seq_len or self.cfg.data.seq_len
        if self.device.type == "cuda":
            seq_len = max(64, seq_len // 64 * 64)
        ds = BinaryDataset.open(data_path)
        loader = DataLoader(ds, seq_len, batch_size, shuffle=False, drop_last=False)
        total_loss, total_tok = 0.0, 0
        for b in loader:
            loss = self.model(b.input.to(self.device), b.target.to(self.device))
            n = b.input.numel()
            total_loss += float(loss) * n
            total_tok += n
            if max_tokens is not None and total_tok >= max_tokens:
                break
        mean = total_loss / max(1, total_tok)
        return {"loss": mean, "perplexity": math.exp(min(mean, 50.0)), "tokens": total_tok}

    @torch.no_grad()
    def evaluate_long_context(self, data_path: str, context_lengths, max_tokens: int = 1 << 20):
        """Perplexity as a function of the context length the model is run at."""
        return {int(L): self.evaluate_perplexity(data_path, max_tokens, seq_len=int(L))
                for L in context_lengths}

    @torch.no_grad()
    def per_token_losses(self, tokens: torch.Tensor) -> torch.Tensor:
        logits = self.model(tokens[:, :-1].to(self.device))
        return K.cross_entropy_rows(logits, tokens[:, 1:].to(self.device)).view(tokens.shape[0], -1)


def sample_top_p(probs: torch.Tensor, top_p: float, generator=None) -> torch.Tensor:
    """Nucleus sampling: smallest set of highest-probability tokens whose mass >= top_p.
    probs: (B, V) -> (B,) token ids."""
    sp, si = torch.sort(probs, dim=-1, descending=True)
    cum = torch.cumsum(sp, dim=-1)
    keep = cum - sp < top_p
    keep[..., 0] = True
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    sp = sp / sp.sum(-1, keepdim=True)
    pick = torch.multinomial(sp, 1, generator=generator)
    return si.gather(-1, pick).squeeze(-1)


class Generator:
    def __init__(self, model: EflaLM, tokenizer=None, seed: int = 0):
        self.model, self.tok = model, tokenizer
        self.device = model.embed_tokens.device
        self.gen = torch.Generator(device=self.device).manual_seed(seed)

    @torch.no_grad()
    def generate_ids(self, prompt_ids, max_new_tokens: int, temperature: float = 1.0,
                     top_p: float = 1.0, eos_id: int | None = None) -> list[int]:
        ids = list(int(t) for t in prompt_ids) or [0]
        states = self.model.new_states(1, self.device)
        logits = None
        for t in ids:  # prefill token by token: the state is all the context there is
            logits = self.model.decode_step(torch.tensor([t], device=self.device), states)
        out = []
        for _ in range(max_new_tokens):
            if temperature <= 0:
                nxt = int(logits.argmax(-1))
            else:
                p = torch.softmax(logits.float() / temperature, -1)
                nxt = int(sample_top_p(p, top_p, self.gen)) if top_p < 1.0 else \
                    int(torch.multinomial(p, 1, generator=self.gen))
            out.append(nxt)
            if eos_id is not None and nxt == eos_id:
                break
            logits = self.model.decode_step(torch.tensor([nxt], device=self.device), states)
        return out

    def generate(self, prompt: str, max_new_tokens: int = 64, temperature: float = 1.0,
                 top_p: float = 0.9) -> str:
        if self.tok is None:
            raise ValueError("a tokenizer is needed to generate from text")
        ids = self.tok.encode(prompt)
        vocab = self.model.cfg.vocab_size
        ids = [i for i in ids if i < vocab]
        new = self.generate_ids(ids, max_new_tokens, temperature, top_p,
                                eos_id=self.tok.special.get("<eos>"))
        return self.tok.decode([t for t in new if t < self.tok.vocab_size()])

    def generate_greedy(self, prompt: str, max_new_tokens: int = 64) -> str:
        return self.generate(prompt, max_new_tokens, temperature=0.0, top_p=1.0)


def benchmark_throughput(model: EflaLM, batch: int, seq_len: int, iters: int = 5,
                         warmup: int = 2) -> dict:
    """Forward-only tokens/s of ``model`` on random tokens (CUDA events on a GPU)."""
    dev = model.embed_tokens.device
    tok = torch.randint(0, model.cfg.vocab_size, (batch, seq_len), device=dev)
    with torch.no_grad():
        for _ in range(warmup):
            model(tok, tok)
        if dev.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(iters):
                model(tok, tok)
            e1.record()
            torch.cuda.synchronize()
            secs = e0.elapsed_time(e1) * 1e-3
        else:
            t0 = time.time()
            for _ in range(iters):
                model(tok, tok)
            secs = time.time() - t0
    return {"tokens_per_second": batch * seq_len * iters / secs, "seconds": secs,
            "batch": batch, "seq_len": seq_len, "iters": iters}
