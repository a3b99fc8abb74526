"""CPU tests: tokenizer, datasets, packing, checkpoint manager, telemetry, formats."""
import json
import os
import urllib.request

import numpy as np
import pytest
import torch

from ceo_b200.data import dataset as D
from ceo_b200.data.synthetic import SyntheticTokens
from ceo_b200.data.tokenizer import Tokenizer, read_token_file
from ceo_b200.runtime.checkpoint import (CheckpointManager, parse_step, read_safetensors)
from ceo_b200.utils import formats
from ceo_b200.utils.telemetry import (HealthStatus, Telemetry, TrainingStats, check_nan_inf)

TEXT = ("the quick brown fox jumps over the lazy dog. the dog barks; the fox runs away.\n"
        "a quick brown dog? no - the quick brown fox!  tabs\tand  double  spaces.\n") * 20


def test_tokenizer_train_encode_decode_roundtrip(tmp_path):
    tok = Tokenizer.train_from_text(TEXT, 300)
    assert tok.vocab_size() == 300 and len(tok.merges) == 40
    assert tok.vocab[256:260] == [b"<pad>", b"<unk>", b"<bos>", b"<eos>"]
    ids = tok.encode(TEXT[:200])
    assert tok.decode(ids) == TEXT[:200] and len(ids) < 200
    assert tok.encode("<eos>") == [259]
    uni = "héllo wörld ✓"
    assert tok.decode(tok.encode(uni)) == uni
    p = tmp_path / "tok.bin"
    tok.save(p)
    t2 = Tokenizer.load(p)
    assert t2.vocab == tok.vocab and t2.merges == tok.merges and t2.encode(TEXT) == tok.encode(TEXT)
    src = tmp_path / "c.txt"
    src.write_text(TEXT)
    n = t2.encode_file(src, tmp_path / "c.tok")
    assert n == len(tok.encode(TEXT))
    assert list(read_token_file(tmp_path / "c.tok")) == tok.encode(TEXT)
    with pytest.raises(ValueError):
        tok.decode([10 ** 6])
    (tmp_path / "bad.bin").write_bytes(b"\0" * 16)
    with pytest.raises(formats.FormatError):
        Tokenizer.load(tmp_path / "bad.bin")


def test_dataset_loader_shards_and_resume(tmp_path):
    toks = np.arange(1000, dtype=np.uint32)
    path = tmp_path / "d.bin"
    D.write_dataset(path, toks)
    ds = D.BinaryDataset.open(path)
    assert len(ds) == 1000 and list(ds.get_tokens(10, 3)) == [10, 11, 12]
    with pytest.raises(IndexError):
        ds.get_tokens(999, 5)
    ld = D.DataLoader(ds, seq_len=16, batch_size=4, shuffle=False)
    b = ld.next()
    assert b.input.shape == (4, 16) and torch.equal(b.target, b.input + 1)
    assert len(ld) == (999 // 16) // 4
    n = 1
    while ld.next() is not None:
        n += 1
    assert n == len(ld)
    # shuffled, data-parallel split is a partition of the windows
    seen = []
    for r in range(2):
        l2 = D.DataLoader(ds, 16, 1, shuffle=True, seed=3, dp_rank=r, dp_world=2)
        seen += [int(x.input[0, 0]) for x in l2]
    assert sorted(seen) == [i * 16 for i in range(62)]
    l3 = D.DataLoader(ds, 16, 2, shuffle=True, seed=9)
    l3.next()
    st = l3.state_dict()
    want = l3.next().input
    l4 = D.DataLoader(ds, 16, 2, shuffle=True, seed=0)
    l4.load_state_dict(st)
    assert torch.equal(l4.next().input, want)
    pf = D.Prefetcher(D.DataLoader(ds, 16, 4, shuffle=False), depth=2)
    assert torch.equal(pf.next().input, b.input)
    pf.close()
    # shards + index + merge
    bld = D.DatasetBuilder(tmp_path / "sh", shard_tokens=300)
    bld.add(toks[:450])
    bld.add(toks[450:])
    idx = bld.finish()
    assert [s.num_tokens for s in bld.shards] == [300, 300, 300, 100]
    with open(idx, "rb") as f:
        ntok, shards, _ = formats.read_dataset_header(f)
    assert ntok == 1000 and shards[1].path == "shard_000001.bin"
    sh1 = D.read_shard(tmp_path / "sh" / "shard_000001.bin")
    assert list(sh1[:2]) == [300, 301]
    import hashlib
    assert hashlib.sha256(sh1.tobytes()).digest() == shards[1].sha256
    bld.merge(tmp_path / "merged.bin")
    assert np.array_equal(D.BinaryDataset.open(tmp_path / "merged.bin").tokens, toks)
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"\x01\x02\x03\x04" * 8)
    with pytest.raises(formats.FormatError):
        D.BinaryDataset.open(bad)


def test_pack_sequences_and_synthetic():
    packs = D.pack_sequences([[1, 2, 3], [4, 5], [6] * 9, [7, 8, 9, 10], [11]], max_len=6)
    assert [p.length for p in packs] == [5, 5]
    assert packs[0].cumulative_lengths == [0, 3, 5] and list(packs[0].sequence_ids[:6]) == \
        [0, 0, 0, 1, 1, -1]
    assert list(packs[1].tokens[:5]) == [7, 8, 9, 10, 11]
    z = SyntheticTokens(1000, "zipf", 1.1, seed=0)
    s = z.sample(20000)
    assert s.min() >= 0 and s.max() < 1000
    counts = np.bincount(s, minlength=1000)
    assert counts[0] > counts[9] > counts[99] and abs(counts[0] / counts[1] - 2 ** 1.1) < 0.4
    assert np.array_equal(SyntheticTokens(1000, "zipf", 1.1, 0).sample(50), s[:50])
    tok, tgt = SyntheticTokens(50, "uniform", seed=1).batch(3, 8)
    assert tok.shape == (3, 8) and torch.equal(tok[:, 1:], tgt[:, :-1])
    with pytest.raises(ValueError):
        SyntheticTokens(10, "gauss")


def test_tensor_file_and_checkpoint_manager(tmp_path):
    tensors = {"a.weight": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int64),
               "s": torch.tensor(2.5)}
    p = tmp_path / "t.bin"
    entries = formats.write_tensor_file(p, tensors)
    assert entries[1].offset == 30 and entries[0].sha256 != formats.EMPTY_SHA256
    back = formats.read_tensor_file(p)
    assert all(torch.equal(back[k], v) for k, v in tensors.items())
    raw = bytearray(p.read_bytes())
    raw[-3] ^= 0xFF
    (tmp_path / "c.bin").write_bytes(raw)
    with pytest.raises(formats.FormatError, match="checksum"):
        formats.read_tensor_file(tmp_path / "c.bin")
    with pytest.raises(formats.FormatError, match="magic"):
        formats.read_tensor_file(p, magic=formats.MAGIC_OPTIMIZER)

    assert parse_step("step_00000042") == 42 and parse_step("step_42") is None
    m = CheckpointManager(tmp_path / "ck", keep_last_n=2, async_save=True)
    for step in (10, 20, 30):
        m.save(step, tensors, {"loss": 1.0 / step, "tokens_seen": step * 100},
               {"master": torch.randn(8)}, b"rngbytes", "model: {}\n", {"scheduler": {"current_step": step}})
    m.wait()
    assert m.list_checkpoints() == [20, 30] and m.latest().endswith("step_00000030")
    md = m.read_metadata(m.latest())
    assert md["step"] == 30 and md["extra"]["scheduler"]["current_step"] == 30
    assert len(md["git_revision"]) == 40 and len(md["config_hash"]) == 64
    assert m.load_rng(m.latest()) == b"rngbytes"
    assert torch.equal(m.load_tensors(m.latest())["b"], tensors["b"])
    assert m.load_optimizer(m.latest())["master"].shape == (8,)
    assert CheckpointManager.validate(m.latest()) == []
    os.remove(os.path.join(m.latest(), "tensors.bin"))
    assert CheckpointManager.validate(m.latest()) == ["missing tensors.bin"]
    # convert
    CheckpointManager.convert(m.path_for(20), tmp_path / "o.safetensors", "safetensors")
    st = read_safetensors(tmp_path / "o.safetensors")
    assert torch.equal(st["a.weight"], tensors["a.weight"])
    CheckpointManager.convert(m.path_for(20), tmp_path / "o.pt", "pytorch")
    assert torch.equal(torch.load(tmp_path / "o.pt")["b"], tensors["b"])
    with pytest.raises(ValueError):
        CheckpointManager.convert(m.path_for(20), tmp_path / "x", "onnx")


class _TinyModel(torch.nn.Module):
    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.a = torch.nn.Parameter(torch.randn(16, 24, generator=g))
        self.b = torch.nn.Parameter(torch.randn(8, 40, generator=g))
        self.n = torch.nn.Parameter(torch.randn(24, generator=g))
        self.s = torch.nn.Parameter(torch.ones(1))


def _flat(world, rank, layout):
    from ceo_b200.optim.flat import FlatParams
    return FlatParams(_TinyModel(), world, rank, layout=layout)


def test_segment_layout_covers_every_parameter_once():
    from ceo_b200.optim.flat import FlatParams
    for world in (1, 2, 4, 8):
        owner = None
        for rank in range(world):
            f = FlatParams(_TinyModel(), world, rank, layout="segment")
            if owner is None:
                owner = torch.full((f.total,), -1, dtype=torch.int64)
            off = 0
            for rg in f.ranges:
                a = rg.goff + rank * rg.len
                assert rg.len % 4 == 0 and rg.goff % 4 == 0 and rg.loff == off
                assert (owner[a:a + rg.len] == -1).all()
                owner[a:a + rg.len] = rank
                off += rg.len
            assert off == f.shard
            # the master shard is the owned slices of the parameters, in shard-local order
            assert torch.equal(f.master, f.owned(f.params).float())
        for seg in f.segments:
            assert (owner[seg.offset:seg.offset + seg.numel] >= 0).all(), seg.name
        # a matrix whose rows divide evenly is split by rows
        rg = f.ranges[f.range_of("a")]
        assert rg.names == ("a",) and rg.len == 16 * 24 // world
    with pytest.raises(ValueError):
        FlatParams(_TinyModel(), 3, 0, layout="segment")


@pytest.mark.parametrize("save_layout,load_layout", [("contiguous", "contiguous"),
                                                      ("segment", "contiguous"),
                                                      ("contiguous", "segment"),
                                                      ("segment", "segment")])
def test_optimizer_resharding_on_load(tmp_path, save_layout, load_layout):
    """Save at world 4, load at world 2: flat-shard tensors are rebuilt through the ownership
    maps, replicated entries come back unchanged, muon entries are the union of all files."""
    flats = [_flat(4, r, save_layout) for r in range(4)]
    total = flats[0].total
    truth = torch.arange(total, dtype=torch.float32) + 1.0
    for r in reversed(range(4)):  # rank 0 last: it waits for the other ranks' markers
        f = flats[r]
        opt = {"master": f.owned(truth), "exp_avg": f.owned(truth * 2),
               "step_count": torch.tensor([5], dtype=torch.int64),
               "side.s.m": torch.tensor([0.25]),
               f"muon.mat{r}.momentum": torch.full((3,), float(r))}
        m = CheckpointManager(tmp_path / "ck", rank=r, world=4)
        m.save(5, {"w": torch.zeros(1)} if r == 0 else {}, {}, opt,
               extra={"flat_layout": f.layout_info()}, shard_timeout=5.0)
    assert CheckpointManager.validate(tmp_path / "ck" / "step_00000005") == []
    for r in range(2):
        f2 = _flat(2, r, load_layout)
        m2 = CheckpointManager(tmp_path / "ck", rank=r, world=2)
        got = m2.load_optimizer(m2.path_for(5), f2)
        assert got["master"].shape == (f2.shard,)
        # every element a parameter occupies comes back where the new map puts it
        want = f2.owned(torch.cat([truth, torch.zeros(max(0, f2.total - total))])[:f2.total])
        covered = f2.owned(_covered_mask(f2))
        assert torch.equal(got["master"][covered], want[covered])
        assert torch.equal(got["exp_avg"][covered], 2 * want[covered])
        assert got["step_count"].tolist() == [5] and got["side.s.m"].tolist() == [0.25]
        assert {k for k in got if k.startswith("muon.")} == \
            {f"muon.mat{i}.momentum" for i in range(4)}


def _covered_mask(f):
    m = torch.zeros(f.total, dtype=torch.bool)
    for seg in f.segments:
        m[seg.offset:seg.offset + seg.numel] = True
    return m


def test_missing_optimizer_shard_is_reported(tmp_path):
    from ceo_b200.utils import errors
    for r in reversed(range(2)):
        m = CheckpointManager(tmp_path / "ck", rank=r, world=2)
        m.save(3, {"w": torch.zeros(1)} if r == 0 else {}, {}, {"master": torch.zeros(4)},
               shard_timeout=5.0)
    path = m.path_for(3)
    (tmp_path / "ck" / "step_00000003" / "optimizer.rank1.bin").unlink()
    assert any("optimizer.rank1.bin" in p for p in CheckpointManager.validate(path))
    with pytest.raises(errors.CheckpointCorrupted):
        CheckpointManager(tmp_path / "ck", rank=1, world=2).load_optimizer(path)
    # rank 0 never commits a checkpoint whose other shards did not arrive
    m0 = CheckpointManager(tmp_path / "ck2", rank=0, world=2)
    with pytest.raises(TimeoutError):
        m0.save(4, {"w": torch.zeros(1)}, {}, {"master": torch.zeros(4)}, shard_timeout=0.3)
    assert m0.latest() is None


def test_telemetry_files_and_prometheus(tmp_path):
    log = tmp_path / "train.log"
    tel = Telemetry(rank=0, log_file=str(log), log_level="debug")
    tel.log_step(3, 300, 1e-4, 0.7)
    tel.log_metrics(3, 2.5, 1e-4, 300, 1234.5, mfu=0.41)
    tel.log("debug", "x", "hello")
    tel.log_health_check(HealthStatus(nan_inf=True))
    port = tel.start_prometheus(0)
    body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
    assert "efla_training_loss 2.5" in body and "efla_tokens_per_second 1234.5" in body
    tel.close()
    rec = json.loads(open(str(log) + ".jsonl").readline())
    assert rec["step"] == 3 and rec["grad_norm"] == 0.7 and set(rec) == \
        {"step", "tokens", "lr", "grad_norm", "timestamp"}
    text = log.read_text()
    assert "step=3 loss=2.5000" in text and "throughput=1234.50" in text and "nan_inf=True" in text
    # non-zero ranks write nothing
    t1 = Telemetry(rank=1, log_file=str(tmp_path / "r1.log"))
    t1.log_step(1, 1, 1.0, 1.0)
    t1.close()
    assert not (tmp_path / "r1.log").exists()
    st = TrainingStats(window=3)
    for i in range(5):
        st.update(float(i), 100, 0.5)
    assert st.avg_loss() == 3.0 and st.tokens_per_sec() == 200.0
    assert check_nan_inf([1.0, float("nan")]) and not check_nan_inf([1.0, 2.0])
    assert not HealthStatus(memory_ok=False).healthy()


def test_aligned_packing_and_state_resets_match_separate_documents():
    """Documents packed on 64-token boundaries with resets give, per document, the loss the
    model gives that document alone."""
    import numpy as np
    import torch
    from ceo_b200.data.dataset import pack_sequences, packed_batch
    from ceo_b200.models.model import EflaLM
    from ceo_b200.utils.config import Config
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = Config.parse_from_file(os.path.join(root, "configs", "smoke_cpu.yaml")).model
    rng = np.random.default_rng(0)
    docs = [rng.integers(1, cfg.vocab_size, size=n) for n in (70, 100, 40, 129)]
    packs = pack_sequences(docs, 321, align=64)
    assert [p.cumulative_lengths for p in packs] == [[0, 70, 228, 296], [0, 129]]
    tokens, targets, resets = packed_batch(packs)
    assert tokens.shape == (2, 320) and resets.tolist() == [[True, False, True, False, True],
                                                            [True, False, False, False, False]]
    model = EflaLM(cfg, "cpu", dtype=torch.float32, seed=0)
    packed = model(tokens, targets, resets=resets)
    # the same documents one by one (each padded to a multiple of 64 with ignored targets)
    num, den = 0.0, 0
    for d in docs:
        T = -(-(len(d) - 1) // 64) * 64
        tok = torch.zeros(1, T, dtype=torch.long)
        tgt = torch.full((1, T), -100, dtype=torch.long)
        tok[0, :len(d) - 1] = torch.from_numpy(d[:-1])
        tgt[0, :len(d) - 1] = torch.from_numpy(d[1:])
        n = len(d) - 1
        num += float(model(tok, tgt)) * n
        den += n
    assert abs(float(packed) - num / den) < 2e-5
    # without the resets the documents leak into each other
    assert abs(float(model(tokens, targets)) - num / den) > 1e-4


def test_bucket_plan_covers_every_ownership_range_once():
    """ZeRO stage 2 / 3: one bucket per transformer block (its matrices, contiguous in the
    ownership map), everything else in the runs reduced after the backward pass."""
    import os

    from ceo_b200.models.model import EflaLM
    from ceo_b200.optim.flat import FlatParams
    from ceo_b200.parallel.fsdp import BucketReducer
    from ceo_b200.utils.config import Config
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = Config.parse_from_file(os.path.join(root, "configs", "smoke_cpu.yaml"))
    cfg.model.num_layers = 3
    model = EflaLM(cfg.model, "cpu", seed=0)
    flat = FlatParams(model, 2, 1, layout="segment")

    class _NoStream:
        pass
    import torch as _t
    orig = _t.cuda.Stream
    _t.cuda.Stream = lambda *a, **k: _NoStream()     # the planner needs no GPU
    try:
        red = BucketReducer(None, flat, [f"blocks.{i}." for i in range(3)])
    finally:
        _t.cuda.Stream = orig
    seen = []
    for b in red.buckets + red.rest:
        assert b is not None
        seen += list(range(*b))
    assert sorted(seen) == list(range(len(flat.ranges)))
    for i, (r0, r1) in enumerate(red.buckets):
        names = [n for rg in flat.ranges[r0:r1] for n in rg.names]
        assert names and all(n.startswith(f"blocks.{i}.") for n in names)
        assert {n.rsplit(".", 1)[-1] for n in names} >= {"w_qkv", "w_o", "w_up", "w_down"}
    rest_names = [n for r0, r1 in red.rest for rg in flat.ranges[r0:r1] for n in rg.names]
    assert "embed_tokens" in rest_names and any(n.endswith("ln1.weight") for n in rest_names)
