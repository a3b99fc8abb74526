"""``efla-train`` command line: train | evaluate | generate | smoke-test | checkpoint |
tokenizer | validate | profile | version | help.

Commands and flags are the reference's (src/main.zig:42-67 dispatch; runTrain 107-157,
runEvaluate 159-196, runGenerate 198-242, runSmokeTest 244-277, runCheckpoint 279-328,
runTokenizer 330-434, runValidate 436-474, runProfile 476-483).  Run as
``python -m ceo_b200.cli <command> ...`` (under ``torchrun`` for more than one GPU).
"""
from __future__ import annotations

import os
import sys

from . import __version__
from .utils.cli_args import ArgParser, CliError
from .utils.config import Config, ConfigError

USAGE = """efla-train <command> [options]

  train        --config C [--resume R] [--data D] [--checkpoint-dir X] [--max-steps N]
  evaluate     --checkpoint P --data D [--config C] [--max-tokens N]
  generate     --checkpoint P --prompt S [--max-tokens N] [--temperature T] [--top-p P]
               [--config C] [--tokenizer T]
  smoke-test   [--config C]
  checkpoint   list --dir D | validate --path P | convert --input I --output O
               --format efla_native|safetensors|pytorch
  tokenizer    train --corpus F --output O [--vocab-size N] [--type bpe]
               | encode --tokenizer T (--text S | --input F) [--output O]
               | decode --tokenizer T --tokens 1,2,3
  validate     --config C
  profile      [--config C --micro-batches N --out F]  (hints, or a per-kernel time table)
  version | help
"""

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _options(args: ArgParser, spec: dict) -> dict:
    """spec: flag -> (kind, default) with kind in str|int|float|flag."""
    out = {k.lstrip("-").replace("-", "_"): d for k, (_, d) in spec.items()}
    while (a := args.next()) is not None:
        if a not in spec:
            raise CliError(f"unknown option {a}")
        kind = spec[a][0]
        key = a.lstrip("-").replace("-", "_")
        if kind == "flag":
            out[key] = True
        elif kind == "int":
            out[key] = args.expect_int(a)
        elif kind == "float":
            out[key] = args.expect_float(a)
        else:
            out[key] = args.expect_string(a)
    return out


def _runtime(cfg=None, log=None):
    """Joins the launched job and looks at the machine (the reference's
    ``DistributedRuntime.init`` + ``Topology.detect``, src/runtime/main.zig:192-240, 322-391):
    device bound, process group up, every rank on Blackwell, peer access between all local
    GPUs checked before any peer-mapped buffer is opened."""
    from .runtime.device import DistributedRuntime, Topology, device_count
    rt = DistributedRuntime.init(None)
    peer_ok = False
    if device_count():
        d = rt.device
        if log:
            free, total = rt.get_memory_info()
            log("info", "runtime", f"rank {rt.rank}/{rt.world_size} on cuda:{rt.local_rank} "
                f"{d.name} sm_{d.major}{d.minor} {d.sm_count} SMs, {free / 2**30:.1f} of "
                f"{total / 2**30:.1f} GiB free")
        if not rt.all_blackwell() and log:
            log("warn", "runtime", "not every rank runs on a Blackwell (sm_100) GPU: the kernel "
                "library is built for sm_100a only")
        if rt.world_size > 1:
            try:
                rt.enable_peer_access()
                peer_ok = True
            except Exception as e:  # noqa: BLE001
                if log:
                    log("warn", "runtime", f"{e}: falling back to library collectives")
        if log and rt.rank == 0:
            try:
                topo = Topology.detect()
                log("info", "runtime", f"topology: {len(topo.numa_nodes)} NUMA node(s), " +
                    ", ".join(f"gpu{a.gpu_id}->numa{a.numa_node}" for a in topo.gpu_affinity))
            except Exception as e:  # noqa: BLE001  (topology is informational)
                log("debug", "runtime", f"topology not available: {e}")
    return rt, peer_ok


def _comm(peer_ok: bool = True):
    from .parallel.comm import Comm, init_distributed
    rank, world, local = init_distributed()
    if world == 1:
        return None
    import torch
    if torch.cuda.is_available() and peer_ok:
        try:
            from .parallel.fused import FusedComm
            return FusedComm()
        except Exception:  # noqa: BLE001
            pass
    return Comm()


def _fit_mesh(rt, world: int):
    """Largest (tp, cp, pp) not above the configured sizes whose product divides ``world``."""
    tp, cp, pp = rt.tensor_parallel_size, rt.context_parallel_size, rt.pipeline_parallel_size
    while world % (tp * cp * pp):
        if pp > 1:
            pp = max(1, pp // 2)
        elif cp > 1:
            cp = max(1, cp // 2)
        elif tp > 1:
            tp = max(1, tp // 2)
        else:
            break
    return tp, cp, pp


def run_train(args: ArgParser) -> int:
    o = _options(args, {"--config": ("str", None), "--resume": ("str", None),
                        "--data": ("str", None), "--checkpoint-dir": ("str", None),
                        "--max-steps": ("int", None)})
    if not o["config"]:
        raise CliError("train: --config is required")
    from .runtime.trainer import Trainer
    from .utils.telemetry import Telemetry
    cfg = Config.parse_from_file(o["config"])
    rt = cfg.runtime
    from .parallel.comm import init_distributed
    rank, world, _ = init_distributed()
    # the mesh of the config (tensor x context x pipeline, data parallel over the rest) must
    # fit the ranks that were launched; a config written for more GPUs is cut down axis by axis
    mp = rt.tensor_parallel_size * rt.context_parallel_size * rt.pipeline_parallel_size
    if world % max(1, mp):
        fitted = _fit_mesh(rt, world)
        print(f"warning: tp x cp x pp = {mp} does not divide {world} rank(s); using "
              f"tp={fitted[0]} cp={fitted[1]} pp={fitted[2]}", file=sys.stderr)
        rt.tensor_parallel_size, rt.context_parallel_size, rt.pipeline_parallel_size = fitted
        mp = fitted[0] * fitted[1] * fitted[2]
    rt.world_size = world
    # the model-parallel engines build their own groups; plain data parallelism gets the
    # peer-memory communicator (library collectives when that is unavailable)
    tel = Telemetry(cfg.telemetry, rank=rank)
    _, peer_ok = _runtime(cfg, tel.log)
    comm = _comm(peer_ok) if mp == 1 else None
    for w in cfg.model.validate():
        tel.log("warn", "config", w)
    cfg.training.validate()
    tr = Trainer(cfg, comm=comm, telemetry=tel, data_path=o["data"],
                 checkpoint_dir=o["checkpoint_dir"])
    if o["resume"]:
        tr.resume(None if o["resume"] == "latest" else o["resume"])
    res = tr.run(o["max_steps"])
    tel.log("info", "trainer", f"done: {res}")
    tel.close()
    return 0


def run_evaluate(args: ArgParser) -> int:
    o = _options(args, {"--checkpoint": ("str", None), "--data": ("str", None),
                        "--config": ("str", None), "--max-tokens": ("int", None)})
    if not o["checkpoint"] or not o["data"]:
        raise CliError("evaluate: --checkpoint and --data are required")
    from .runtime.evaluator import Evaluator, load_model
    cfg = Config.parse_from_file(o["config"]) if o["config"] else None
    model, cfg = load_model(o["checkpoint"], cfg)
    res = Evaluator(model, cfg).evaluate_perplexity(o["data"], o["max_tokens"])
    print(f"loss={res['loss']:.6f} perplexity={res['perplexity']:.4f} tokens={res['tokens']}")
    return 0


def run_generate(args: ArgParser) -> int:
    o = _options(args, {"--checkpoint": ("str", None), "--prompt": ("str", ""),
                        "--max-tokens": ("int", 64), "--temperature": ("float", 1.0),
                        "--top-p": ("float", 0.9), "--config": ("str", None),
                        "--tokenizer": ("str", None)})
    if not o["checkpoint"]:
        raise CliError("generate: --checkpoint is required")
    from .data.tokenizer import Tokenizer
    from .runtime.evaluator import Generator, load_model
    cfg = Config.parse_from_file(o["config"]) if o["config"] else None
    model, cfg = load_model(o["checkpoint"], cfg)
    tpath = o["tokenizer"] or cfg.data.tokenizer_path
    if os.path.exists(tpath):
        tok = Tokenizer.load(tpath)
    else:
        tok = Tokenizer()  # byte-level fallback: ids 0..255 are the raw bytes
    text = Generator(model, tok, cfg.runtime.seed).generate(o["prompt"], o["max_tokens"],
                                                            o["temperature"], o["top_p"])
    print(text)
    return 0


def run_smoke_test(args: ArgParser) -> int:
    o = _options(args, {"--config": ("str", os.path.join(ROOT, "configs", "smoke.yaml"))})
    from .runtime.trainer import Trainer
    cfg = Config.parse_from_file(o["config"])
    cfg.runtime.world_size = 1
    cfg.runtime.tensor_parallel_size = 1
    tr = Trainer(cfg)
    losses = tr.smoke_test()
    ok = all(l == l for l in losses)
    print(f"smoke test {'passed' if ok else 'FAILED'}: losses {losses}")
    return 0 if ok else 1


def run_checkpoint(args: ArgParser) -> int:
    from .runtime.checkpoint import CheckpointManager
    sub = args.next()
    if sub == "list":
        o = _options(args, {"--dir": ("str", "checkpoints")})
        m = CheckpointManager(o["dir"])
        for s in m.list_checkpoints():
            md = m.read_metadata(m.path_for(s))
            print(f"step_{s:08d} loss={md.get('loss', 0):.4f} tokens={md.get('tokens_seen', 0)}")
        return 0
    if sub == "validate":
        o = _options(args, {"--path": ("str", None)})
        if not o["path"]:
            raise CliError("checkpoint validate: --path is required")
        problems = CheckpointManager.validate(o["path"])
        for p in problems:
            print(f"invalid: {p}")
        print("checkpoint valid" if not problems else "checkpoint INVALID")
        return 0 if not problems else 1
    if sub == "convert":
        o = _options(args, {"--input": ("str", None), "--output": ("str", None),
                            "--format": ("str", "safetensors")})
        if not o["input"] or not o["output"]:
            raise CliError("checkpoint convert: --input and --output are required")
        CheckpointManager.convert(o["input"], o["output"], o["format"])
        print(f"wrote {o['output']} ({o['format']})")
        return 0
    raise CliError("checkpoint: expected list | validate | convert")


def run_tokenizer(args: ArgParser) -> int:
    from .data.tokenizer import Tokenizer
    sub = args.next()
    if sub == "train":
        o = _options(args, {"--corpus": ("str", None), "--output": ("str", "tokenizer.bin"),
                            "--vocab-size": ("int", 8192), "--type": ("str", "bpe")})
        if not o["corpus"]:
            raise CliError("tokenizer train: --corpus is required")
        if o["type"] != "bpe":
            raise CliError(f"tokenizer type {o['type']!r} is not implemented (only bpe)")
        tok = Tokenizer.train(o["corpus"], o["vocab_size"])
        tok.save(o["output"])
        print(f"trained {tok.vocab_size()} tokens ({len(tok.merges)} merges) -> {o['output']}")
        return 0
    if sub == "encode":
        o = _options(args, {"--tokenizer": ("str", None), "--text": ("str", None),
                            "--input": ("str", None), "--output": ("str", None)})
        if not o["tokenizer"]:
            raise CliError("tokenizer encode: --tokenizer is required")
        tok = Tokenizer.load(o["tokenizer"])
        if o["input"]:
            out = o["output"] or o["input"] + ".tokens"
            n = tok.encode_file(o["input"], out)
            print(f"{n} tokens -> {out}")
        elif o["text"] is not None:
            print(" ".join(str(t) for t in tok.encode(o["text"])))
        else:
            raise CliError("tokenizer encode: --text or --input is required")
        return 0
    if sub == "decode":
        o = _options(args, {"--tokenizer": ("str", None), "--tokens": ("str", None)})
        if not o["tokenizer"] or o["tokens"] is None:
            raise CliError("tokenizer decode: --tokenizer and --tokens are required")
        tok = Tokenizer.load(o["tokenizer"])
        ids = [int(x) for x in o["tokens"].replace(",", " ").split()]
        print(tok.decode(ids))
        return 0
    raise CliError("tokenizer: expected train | encode | decode")


def run_validate(args: ArgParser) -> int:
    o = _options(args, {"--config": ("str", None)})
    if not o["config"]:
        raise CliError("validate: --config is required")
    cfg = Config.parse_from_file(o["config"])
    warns = cfg.model.validate()
    cfg.training.validate()
    cfg.runtime.validate()
    for w in warns:
        print(f"warning: {w}")
    print(f"Estimated memory per GPU: {cfg.model.estimate_memory() / 2**30:.2f} GB")
    n = cfg.model.count_parameters()
    print(f"Total parameters: {n}")
    if not 0.95 <= n / 1e12 <= 1.05:
        print("warning: parameter count differs from the 1T target by more than 5%")
    print("Configuration valid!")
    return 0


def run_profile(args: ArgParser) -> int:
    """Without --config: how to profile.  With --config on a GPU machine: one training step of
    that config under the in-process profiler, as a per-kernel time table (a diagnostic, not a
    benchmark: bench.py times without any profiler)."""
    o = _options(args, {"--config": ("str", None), "--micro-batches": ("int", 2),
                        "--out": ("str", None)})
    hints = ("Timing: python bench.py --gpus 1 (CUDA events, device-timed)\n"
             "Per-kernel roofline: python -m ceo_b200.utils.kernel_bench --torch\n"
             "Launch list: ncu --metrics gpu__time_duration.sum --clock-control none -c 4000 --csv "
             "python bench.py --steps 1 --warmup 1 --global-batch 4 --skip-e2e\n"
             "One kernel in depth: ncu --set full --clock-control none -k regex:<kernel> -c 3 "
             "-o prof <small command>\n"
             "Timeline ranges: CEO_TRACE=1 puts NVTX ranges around forward / backward / optimizer")
    import torch
    if not o.get("config") or not torch.cuda.is_available():
        print(hints)
        return 0
    from .data.synthetic import SyntheticTokens
    from .runtime.engine import TrainEngine
    from .utils import tracing
    cfg = Config.parse_from_file(o["config"])
    cfg.runtime.world_size, cfg.runtime.tensor_parallel_size = 1, 1
    dev = torch.device("cuda", 0)
    eng = TrainEngine(cfg, dev, None)
    data = SyntheticTokens(cfg.model.vocab_size, cfg.data.synthetic.kind or "zipf",
                           cfg.data.synthetic.s, cfg.data.synthetic.seed, 0)
    mb = [tuple(t.to(dev) for t in data.batch(cfg.training.micro_batch_size, cfg.data.seq_len))
          for _ in range(int(o["micro_batches"]))]
    text = tracing.format_table(tracing.kernel_table(lambda: eng.train_step(mb, 1e-4)))
    print(text)
    if o.get("out"):
        with open(o["out"], "w") as f:
            f.write(text + "\n")
    return 0


COMMANDS = {"train": run_train, "evaluate": run_evaluate, "generate": run_generate,
            "smoke-test": run_smoke_test, "checkpoint": run_checkpoint,
            "tokenizer": run_tokenizer, "validate": run_validate, "profile": run_profile}


def main(argv=None) -> int:
    args = ArgParser(sys.argv[1:] if argv is None else argv)
    cmd = args.next()
    if cmd in (None, "help", "--help", "-h"):
        print(USAGE)
        return 0
    if cmd in ("version", "--version"):
        print(f"efla-train (ceo_b200) {__version__}")
        return 0
    fn = COMMANDS.get(cmd)
    if fn is None:
        print(f"unknown command {cmd!r}\n\n{USAGE}", file=sys.stderr)
        return 2
    try:
        return fn(args)
    except (CliError, ConfigError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
