"""bf16 against FP8 training on the same data and seed: is ``training.fp8_training`` safe to
switch on for a model?

    python -m ceo_b200.utils.fp8_convergence --config configs/efla_340m.yaml --steps 200

trains the config's model twice on one GPU from the same initial weights and the same
synthetic token stream - once in bf16, once with the projections' forward, data-gradient and
weight-gradient GEMMs on 8-bit operands (delayed scaling, ``--margin`` bits of headroom) - with
the config's learning-rate schedule, and prints the loss of both runs every ``--every`` steps
and the mean gap over the last tenth of the run as one JSON record.  The batch is cut down
(``--global-batch``, ``--seq-len``) so that a few hundred optimizer steps take a minute.

The reference has the switch (``training.fp8_training``, src/util/config.zig:420) and the
codecs (src/tensor/dtype.zig:203-264) but no training path that uses them, so there is nothing
of its own to compare against.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..data.synthetic import SyntheticTokens
from ..runtime.engine import TrainEngine
from .config import Config


def run(cfg_path: str, fp8: bool, steps: int, gbs: int, seq: int, margin: int, every: int):
    cfg = Config.parse_from_file(cfg_path)
    cfg.runtime.world_size = 1
    cfg.data.seq_len = seq or cfg.data.seq_len
    cfg.training.global_batch_size = gbs
    cfg.training.micro_batch_size = min(cfg.training.micro_batch_size, gbs)
    cfg.training.total_steps = steps
    cfg.training.warmup_steps = min(cfg.training.warmup_steps, max(1, steps // 10))
    cfg.training.fp8_training = fp8
    cfg.training.fp8_gradients = fp8
    dev = torch.device("cuda", torch.cuda.current_device())
    eng = TrainEngine(cfg, dev, None, seed=cfg.runtime.seed)
    if eng.fp8 is not None and margin >= 0:
        eng.fp8.margin = margin
        for st in eng.fp8.states:
            for m in (st.x_meta, st.w_meta, st.g_meta):
                m.margin = margin
    data = SyntheticTokens(cfg.model.vocab_size, cfg.data.synthetic.kind or "zipf",
                           cfg.data.synthetic.s, cfg.data.synthetic.seed, 0)
    mbs = cfg.training.micro_batch_size
    n_micro = gbs // mbs
    losses = []
    for step in range(steps):
        mb = [tuple(t.to(dev) for t in data.batch(mbs, cfg.data.seq_len)) for _ in range(n_micro)]
        loss, _ = eng.train_step(mb)
        losses.append(loss)
        if every and (step + 1) % every == 0:
            print(json.dumps({"run": "fp8" if fp8 else "bf16", "step": step + 1,
                              "loss": round(float(loss), 4)}), flush=True)
    out = [float(x) for x in losses]
    del eng
    torch.cuda.empty_cache()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--global-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--margin", type=int, default=-1, help="FP8 headroom bits (default: engine's)")
    ap.add_argument("--every", type=int, default=25)
    a = ap.parse_args(argv)
    ref = run(a.config, False, a.steps, a.global_batch, a.seq_len, a.margin, a.every)
    f8 = run(a.config, True, a.steps, a.global_batch, a.seq_len, a.margin, a.every)
    tail = max(1, a.steps // 10)
    m_ref = sum(ref[-tail:]) / tail
    m_f8 = sum(f8[-tail:]) / tail
    rec = {"config": a.config, "steps": a.steps, "global_batch": a.global_batch,
           "loss_first": [round(ref[0], 4), round(f8[0], 4)],
           "loss_last_tenth_bf16": round(m_ref, 4), "loss_last_tenth_fp8": round(m_f8, 4),
           "gap": round(m_f8 - m_ref, 4), "rel_gap": round((m_f8 - m_ref) / m_ref, 5),
           "max_abs_gap": round(max(abs(x - y) for x, y in zip(ref, f8)), 4)}
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
