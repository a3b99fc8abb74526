"""CPU unit tests: YAML, config, hashing, RNG, dtype codecs, layout, sharding, CLI args."""
import math

import numpy as np
import pytest
import torch

from ceo_b200.parallel import sharding as sh
from ceo_b200.utils import cli_args, dtypes, errors, hashing, layout, rng, yaml_compat
from ceo_b200.utils.config import Config, ConfigError


def test_yaml_scalars_and_nesting():
    doc = yaml_compat.loads("""
# comment
a: 1
b: 0x10
c: 1.5e-3
d: true
e: no
f: ~
g: "quoted # not comment"
h: 12abc
nested:
  x: -3
  deeper:
    y: 'z'
list:
  - 1
  - two
  - 3.0
inline: [1, 2, x]
maps:
\t- name: a
\t  v: 1
\t- name: b
""")
    assert doc["a"] == 1 and doc["b"] == 16 and doc["c"] == 1.5e-3
    assert doc["d"] is True and doc["e"] is False and doc["f"] is None
    assert doc["g"] == "quoted # not comment" and doc["h"] == "12abc"
    assert doc["nested"]["deeper"]["y"] == "z" and doc["nested"]["x"] == -3
    assert doc["list"] == [1, "two", 3.0] and doc["inline"] == [1, 2, "x"]
    assert doc["maps"] == [{"name": "a", "v": 1}, {"name": "b"}]
    assert yaml_compat.parse_scalar("1e5") == 1e5 and yaml_compat.parse_scalar("15") == 15
    assert yaml_compat.loads(yaml_compat.dumps(doc)) == doc


def test_config_defaults_sections_and_validation():
    full = {s: {} for s in ("model", "training", "runtime", "data", "checkpoint", "telemetry")}
    cfg = Config.from_dict(full)
    assert cfg.model.hidden_dim == 16384 and cfg.training.optimizer == "lion_muon"
    assert cfg.runtime.zero_stage == 2 and cfg.data.seq_len == 8192
    assert cfg.checkpoint.keep_last_n == 5 and cfg.telemetry.prometheus_port == 9090
    assert cfg.model.efla.chunk_size == 4096 and cfg.model.prism.shortconv_window == 64
    with pytest.raises(ConfigError):
        Config.from_dict({"model": {}})
    bad = dict(full, training={"global_batch_size": 7, "micro_batch_size": 2})
    with pytest.raises(ConfigError):
        Config.from_dict(bad).training.validate()
    with pytest.raises(ConfigError):
        Config.from_dict(dict(full, model={"activation": "nope"})).model.validate()
    with pytest.raises(ConfigError):
        Config.from_dict(dict(full, model={"hidden_dim": "x"}))
    assert Config.from_yaml(cfg.to_yaml()) == cfg
    assert len(cfg.config_hash()) == 32
    # unknown keys are ignored
    assert Config.from_dict(dict(full, model={"bogus": 1})).model.vocab_size == 65536


def test_shipped_configs_parse():
    import glob
    import os
    root = os.path.join(os.path.dirname(os.path.dirname(__file__)), "configs")
    files = glob.glob(os.path.join(root, "*.yaml"))
    assert len(files) >= 6
    for f in files:
        cfg = Config.parse_from_file(f)
        cfg.model.validate()
        cfg.training.validate()
    c = Config.parse_from_file(os.path.join(root, "efla_1p3b.yaml"))
    assert (c.model.hidden_dim, c.model.num_layers, c.model.num_heads, c.model.head_dim,
            c.model.intermediate_dim, c.model.vocab_size, c.data.seq_len) == \
        (2048, 24, 16, 128, 5632, 32000, 4096)
    assert c.training.global_batch_size * c.data.seq_len == 1 << 20
    # the accumulation count written in the file is the one the batch sizes imply on 8 GPUs,
    # and every GPU count of the scaling run divides the global batch into whole micro-batches
    t = c.training
    assert t.gradient_accumulation_steps * t.micro_batch_size * c.runtime.world_size == \
        t.global_batch_size
    for n in (1, 2, 4, 8):
        assert t.global_batch_size % (t.micro_batch_size * n) == 0


def test_hashing():
    assert hashing.to_hex(hashing.sha256(b"abc")).startswith("ba7816bf")
    assert hashing.verify(b"abc", hashing.sha256(b"abc"))
    assert hashing.xxhash64(b"") == 0xEF46DB3751D8E999
    assert hashing.xxhash64(b"abc") == 0x44BC2CF5AD770999
    assert hashing.combine_hash(1, 2) != hashing.combine_hash(2, 1)
    assert hashing.hash_string("x") == hashing.xxhash64(b"x")


def test_rng_determinism_and_distribution():
    a, b = rng.DeterministicRng(7), rng.DeterministicRng(7)
    assert [a.next_u32() for _ in range(5)] == [b.next_u32() for _ in range(5)]
    assert rng.DeterministicRng(8).next_u32() != rng.DeterministicRng(7).next_u32()
    r = rng.DeterministicRng(1)
    xs = [r.float() for _ in range(4000)]
    assert 0 <= min(xs) and max(xs) < 1 and abs(sum(xs) / len(xs) - 0.5) < 0.03
    ns = [r.float_norm() for _ in range(4000)]
    assert abs(sum(ns) / len(ns)) < 0.06 and abs(np.std(ns) - 1) < 0.06
    assert all(3 <= r.int_range(3, 9) < 9 for _ in range(200))
    items = list(range(50))
    r.shuffle(items)
    assert sorted(items) == list(range(50)) and items != list(range(50))
    d0, d1 = rng.DistributedRng(5, 0), rng.DistributedRng(5, 1)
    assert d0["data"].next_u32() != d1["data"].next_u32()
    st = d0.state_bytes()
    nxt = d0["init"].next_u32()
    d0.load_state_bytes(st)
    assert d0["init"].next_u32() == nxt
    p = rng.PhiloxRng(123)
    assert p.block(5) == rng.PhiloxRng(123).block(5) and p.block(5) != p.block(6)
    f = r.fork()
    assert f.next_u32() != r.next_u32()


def test_dtype_codecs_roundtrip():
    x = np.array([0.0, 1.0, -1.5, 3.14159, 1e-3, 448.0, 1e6, -1e6, np.inf, np.nan], np.float32)
    bf = dtypes.bf16_bits_to_f32(dtypes.f32_to_bf16_bits(x))
    tb = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(bf[:-1], tb[:-1]) and np.isnan(bf[-1])
    h = dtypes.fp16_bits_to_f32(dtypes.f32_to_fp16_bits(x[:6]))
    assert np.allclose(h, x[:6], rtol=1e-3, atol=1e-6)
    e4 = dtypes.FP8_E4M3.decode(dtypes.FP8_E4M3.encode(x))
    t4 = torch.from_numpy(np.nan_to_num(x[:8], posinf=448, neginf=-448)).clamp(-448, 448) \
        .to(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(e4[:8], t4) and e4[8] == 448.0 and np.isnan(e4[9])
    e5 = dtypes.FP8_E5M2.decode(dtypes.FP8_E5M2.encode(x[:6]))
    t5 = torch.from_numpy(x[:6]).to(torch.float8_e5m2).float().numpy()
    assert np.array_equal(e5, t5)
    # every code survives decode -> encode; subnormals included
    codes = np.arange(256, dtype=np.uint8)
    v = dtypes.FP8_E4M3.decode(codes)
    ok = ~np.isnan(v)
    assert np.array_equal(dtypes.FP8_E4M3.encode(v[ok]) & 0x7F, codes[ok] & 0x7F)
    vals = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -6, -0.5], np.float32)
    assert np.array_equal(dtypes.fp4_unpack(dtypes.fp4_pack(vals), vals.size), vals)
    out = dtypes.cast_slice(dtypes.encode(vals, dtypes.DType.bf16), dtypes.DType.bf16,
                            dtypes.DType.fp16)
    assert np.array_equal(dtypes.decode(out, dtypes.DType.fp16), vals)
    assert dtypes.DType.fp8_e4m3.bit_size() == 8 and dtypes.DType.fp4.is_quantized()
    assert dtypes.DType.bf16.accumulation_dtype() == dtypes.DType.fp32
    sf = dtypes.ScaleFactor()
    assert sf.update(2.0) == 224.0 and sf.update(1.0) == 224.0
    for _ in range(16):
        sf.update(1.0)
    assert sf.scale == 448.0
    bs = dtypes.BlockScale(8)
    y = np.linspace(-3, 3, 20).astype(np.float32)
    q, s = bs.quantize(y)
    assert np.allclose(bs.dequantize(q, s, 20), y, rtol=0.07, atol=1e-3)


def test_layout_and_pool():
    assert layout.pad_dimension(13, 8) == 16 and layout.optimal_leading_dimension(100) == 104
    t = layout.TensorCoreTiles()
    assert (t.M, t.N, t.K) == (128, 256, 64)
    pool = layout.MemoryPool(4096, device="cpu")
    a = pool.allocate((10, 10), torch.float32)
    b = pool.allocate((7,), torch.bfloat16)
    assert a.shape == (10, 10) and b.data_ptr() % 2 == 0 and pool.used() >= 414
    with pytest.raises(MemoryError):
        pool.allocate((4096,), torch.float32)
    pool.reset()
    assert pool.used() == 0


def test_sharding_math_and_rank_mapping():
    s = [sh.ShardSpec(0, 3, i) for i in range(3)]
    assert [x.local_shape((10, 4)) for x in s] == [(4, 4), (3, 4), (3, 4)]
    assert [x.global_offset((10, 4))[0] for x in s] == [0, 4, 7]
    assert sh.ShardSpec.no_sharding().local_shape((5, 5)) == (5, 5)
    with pytest.raises(sh.ParallelError):
        sh.ShardSpec(0, 2, 2)
    with pytest.raises(sh.ParallelError):
        sh.ShardSpec(3, 2, 0).local_shape((4, 4))
    full = torch.arange(40).view(10, 4)
    assert torch.equal(torch.cat([x.slice_of(full) for x in s]), full)
    tp = sh.TensorParallelConfig(4, 1)
    assert tp.spec("qkv").shard_dim == 0 and tp.spec("attn_out").shard_dim == 1
    sp = sh.SequenceParallelConfig(4, 3)
    assert sp.local_seq_len(10) == 2 and sp.seq_offset(10) == 8
    z = sh.ZeroConfig.for_stage(2)
    assert z.partition_gradients and not z.partition_params
    assert z.owns_parameter(3 << 20, 3, 8) and not z.owns_parameter(3 << 20, 2, 8)
    seen = set()
    for r in range(16):
        pc = sh.ParallelConfig.from_global_rank(r, 2, 2, 2, 2)
        assert pc.global_rank() == r
        seen.add((pc.pp_rank, pc.dp_rank, pc.tp_rank, pc.sp_rank))
    assert len(seen) == 16
    pc = sh.ParallelConfig.from_global_rank(5, 1, 2, 4, 1)
    assert (pc.dp_rank, pc.tp_rank) == (1, 1) and pc.group_ranks("tp") == [4, 5, 6, 7]
    assert pc.group_ranks("dp") == [1, 5] and pc.global_world_size() == 8


def test_cli_args_and_errors():
    a = cli_args.ArgParser(["--x", "5", "--f", "--k=v", "1.5"])
    assert a.parse_option("--x") == "5" and a.parse_flag("--f") and a.parse_option("--k") == "v"
    assert a.peek() == "1.5" and a.expect_float() == 1.5 and a.next() is None
    with pytest.raises(cli_args.CliError):
        cli_args.ArgParser(["z"]).expect_int()
    assert cli_args.parse_key_value("a=b, c=d") == {"a": "b", "c": "d"}
    assert errors.check_finite(1.0) == 1.0
    with pytest.raises(errors.NaNDetected):
        errors.check_finite(math.nan)
    with pytest.raises(errors.InfDetected):
        errors.check_finite_slice([1.0, math.inf])
    assert "step 3" in str(errors.ErrorContext(ValueError("x"), "forward", 3, 1))


def test_tensor_ops_cpu_paths():
    import torch
    from ceo_b200.ops import tensor_ops as T
    x = torch.arange(1, 6, dtype=torch.float32)[None]
    assert T.cumsum(x).tolist() == [[1, 3, 6, 10, 15]]
    assert T.cumsum(x, exclusive=True).tolist() == [[0, 1, 3, 6, 10]]
    assert T.cumsum(x, reverse=True).tolist() == [[15, 14, 12, 9, 5]]
    assert T.cumsum(x, True, True).tolist() == [[14, 12, 9, 5, 0]]
    src = torch.arange(12.).view(3, 4)
    out = T.gather_rows(src, torch.tensor([2, -1, 0, 5]))
    assert out.tolist() == [[8, 9, 10, 11], [0] * 4, [0, 1, 2, 3], [0] * 4]
    dst = torch.zeros(3, 4)
    T.scatter_add_rows(dst, torch.tensor([1, 1, 7]), torch.ones(3, 4))
    assert dst[1].tolist() == [2.0] * 4 and dst.sum().item() == 8.0
    assert T.transpose2d(src.bfloat16()).shape == (4, 3)


def test_topology_from_fake_nvml_and_sysfs(tmp_path):
    from ceo_b200.runtime.device import DeviceInfo, Topology, parse_cpulist
    assert parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    for nid, cpus in ((0, "0-3"), (1, "4-7")):
        d = tmp_path / "devices" / "system" / "node" / f"node{nid}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpus + "\n")
        (d / "meminfo").write_text(f"Node {nid} MemTotal:       1024 kB\n")
    for bdf, node in (("0000:1b:00.0", 0), ("0000:9d:00.0", 1)):
        d = tmp_path / "bus" / "pci" / "devices" / bdf
        d.mkdir(parents=True)
        (d / "numa_node").write_text(f"{node}\n")

    class FakeNvml:
        def count(self): return 2
        def pci(self, i): return (0, (0x1b, 0x9d)[i], 0, ("00000000:1B:00.0", "00000000:9D:00.0")[i])
        def nvlinks(self, i): return 18

    t = Topology.detect(nvml=FakeNvml(), sysfs=str(tmp_path))
    assert [n.gpus for n in t.numa_nodes] == [[0], [1]]
    assert t.numa_nodes[1].cpus == [4, 5, 6, 7] and t.numa_nodes[0].memory_size == 1024 * 1024
    assert t.gpu_affinity[1].pci_bus == 0x9d and t.gpu_affinity[1].nvlink_active == 18
    assert t.gpu_for_numa(1) == 1 and t.gpu_for_numa(5) is None
    assert t.cpus_for_gpu(0) == [0, 1, 2, 3]
    # no sources at all: one node, bus = index (all the reference reports)
    class NoNvml:
        def count(self): return 3
        def pci(self, i): raise RuntimeError
        def nvlinks(self, i): return 0
    t = Topology.detect(nvml=NoNvml(), sysfs=str(tmp_path / "nowhere"))
    assert len(t.numa_nodes) == 1 and t.numa_nodes[0].gpus == [0, 1, 2]
    assert [a.pci_bus for a in t.gpu_affinity] == [0, 1, 2]
    assert DeviceInfo(0, "B200", 10, 0, 148, 1).is_blackwell
    assert not DeviceInfo(0, "H100", 9, 0, 132, 1).is_blackwell


def test_runtime_queries_without_a_gpu_and_tracing_noop():
    import pytest
    import torch
    from ceo_b200.parallel.pipeline import stage_bounds
    from ceo_b200.runtime import device
    from ceo_b200.utils import errors, tracing
    if not torch.cuda.is_available():
        assert device.device_count() == 0
        with pytest.raises(errors.NoGpuAvailable):
            device.device_info(0)
        with pytest.raises(errors.NoGpuAvailable):
            device.DistributedRuntime.init_single_gpu()
        assert device.peer_access_matrix(0) == []
    # uneven layer split: the first stages take the remainder
    assert [stage_bounds(10, 4, s) for s in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [stage_bounds(2, 4, s) for s in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    # ranges are no-ops when tracing is off or there is no GPU
    tracing.set_enabled(True)
    with tracing.trace_range("x"):
        pass
    tracing.set_enabled(False)
    assert not tracing.enabled()
    t = tracing.format_table({"busy_ms": 2.0, "span_ms": 2.5, "kernels": [("k", 3, 1.5), ("j", 1, 0.5)]})
    assert "75.0%" in t and "k" in t


def test_normal_build_has_no_bounds_checks_compiled_in():
    from ceo_b200.ops import _lib
    if not _lib.available():
        pytest.skip("kernel library not built")
    assert not _lib.BOUNDS_CHECK
    assert _lib.bounds_status() is None
    assert _lib.lib().ceo_bounds_selftest(None, 4, 1, None) == -1
