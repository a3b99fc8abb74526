"""Configuration schema: the reference's six-section YAML (src/util/config.zig:4-683)
as dataclasses with the same keys, defaults, enum strings and validation rules.

All six sections (model, training, runtime, data, checkpoint, telemetry) must be present
(config.zig:32-37); unknown keys are ignored and missing keys take their defaults.
Extensions (all defaulting to the reference's behaviour):
``runtime.context_parallel_size``, ``runtime.data_parallel_size`` (derived when 0),
``model.efla.{use_query, per_token_beta, normalize_qk}``, ``training.adam_{beta1,beta2,eps}``,
``data.synthetic: {kind: uniform|zipf, s, seed}``.
"""
from __future__ import annotations

import dataclasses
import hashlib
from dataclasses import dataclass, field, fields
from typing import Any

from . import yaml_compat

NORM_TYPES = ("layernorm", "rmsnorm")
ACTIVATIONS = ("relu", "gelu", "silu", "swiglu")
BETA_SCHEDULES = ("constant", "linear_warmup", "cosine_decay")
OPTIMIZERS = ("lion", "muon", "lion_muon", "adamw")
LR_SCHEDULES = ("constant", "linear_warmup", "cosine", "linear_warmup_cosine")
LOG_LEVELS = ("debug", "info", "warn", "err")
DTYPES = ("fp32", "fp16", "bf16", "fp8")


class ConfigError(ValueError):
    pass


def _coerce(value: Any, default: Any, name: str):
    if value is None:
        return default
    if isinstance(default, bool):
        if isinstance(value, bool):
            return value
        raise ConfigError(f"{name}: expected a boolean, got {value!r}")
    if isinstance(default, int) and not isinstance(default, bool):
        if isinstance(value, bool):
            raise ConfigError(f"{name}: expected an integer, got {value!r}")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value == int(value):
            return int(value)
        raise ConfigError(f"{name}: expected an integer, got {value!r}")
    if isinstance(default, float):
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        raise ConfigError(f"{name}: expected a number, got {value!r}")
    if isinstance(default, str):
        return str(value)
    return value


def _from_map(cls, m: dict | None, path: str):
    m = m or {}
    if not isinstance(m, dict):
        raise ConfigError(f"{path}: expected a map")
    kw = {}
    for f in fields(cls):
        if f.default_factory is not dataclasses.MISSING and \
                dataclasses.is_dataclass(f.default_factory):
            kw[f.name] = _from_map(f.default_factory, m.get(f.name), f"{path}.{f.name}")
        else:
            default = f.default if f.default is not dataclasses.MISSING else f.default_factory()
            kw[f.name] = _coerce(m.get(f.name), default, f"{path}.{f.name}")
    obj = cls(**kw)
    return obj


def _enum(value: str, allowed, name: str) -> str:
    if value not in allowed:
        raise ConfigError(f"{name}: {value!r} is not one of {', '.join(allowed)}")
    return value


@dataclass
class EflaConfig:  # config.zig:254-305
    enabled: bool = True
    num_heads: int = 128
    state_dim: int = 128
    chunk_size: int = 4096
    learned_beta: bool = True
    initial_beta: float = 1.0
    beta_schedule: str = "constant"
    use_chunked_scan: bool = True
    # extensions
    use_query: bool = False
    per_token_beta: bool = False
    normalize_qk: bool = False


@dataclass
class PrismConfig:  # config.zig:314-353
    enabled: bool = True
    num_iterations: int = 3
    shortconv_window: int = 64
    use_proxy: bool = True
    forget_factor: float = 0.99


@dataclass
class ModelConfig:  # config.zig:62-231
    name: str = "efla-1t"
    vocab_size: int = 65536
    hidden_dim: int = 16384
    num_layers: int = 80
    num_heads: int = 128
    num_kv_heads: int = 16
    head_dim: int = 128
    intermediate_dim: int = 65536
    max_seq_len: int = 50000000
    norm_type: str = "rmsnorm"
    activation: str = "gelu"
    tie_embeddings: bool = False
    dropout: float = 0.0
    dtype: str = "bf16"
    target_params: int = 1000000000000
    efla: EflaConfig = field(default_factory=EflaConfig)
    prism: PrismConfig = field(default_factory=PrismConfig)

    def validate(self) -> list[str]:
        """Raises on structural errors; returns warnings (parameter count vs target_params
        outside +-5 %, config.zig:155-171)."""
        if self.hidden_dim <= 0:
            raise ConfigError("model.hidden_dim must be positive")
        if self.num_layers <= 0:
            raise ConfigError("model.num_layers must be positive")
        if self.num_heads <= 0:
            raise ConfigError("model.num_heads must be positive")
        if self.head_dim <= 0:
            raise ConfigError("model.head_dim must be positive")
        if self.hidden_dim % self.num_heads != 0:
            raise ConfigError("model.hidden_dim must be divisible by model.num_heads")
        _enum(self.norm_type, NORM_TYPES, "model.norm_type")
        _enum(self.activation, ACTIVATIONS, "model.activation")
        _enum(self.dtype, DTYPES, "model.dtype")
        _enum(self.efla.beta_schedule, BETA_SCHEDULES, "model.efla.beta_schedule")
        warns = []
        ratio = self.count_parameters() / max(1, self.target_params)
        if ratio < 0.95:
            warns.append(f"parameter count {self.count_parameters()} is below target "
                         f"{self.target_params} by more than 5%")
        elif ratio > 1.05:
            warns.append(f"parameter count {self.count_parameters()} exceeds target "
                         f"{self.target_params} by more than 5%")
        return warns

    def count_layer_parameters(self) -> int:
        """The reference's per-layer estimate (config.zig:196-217): q + kv-head projections,
        output projection, PRISM projections, a two-matrix MLP, two norms."""
        p = self.hidden_dim * (self.hidden_dim + 2 * self.num_kv_heads * self.head_dim)
        p += self.hidden_dim * self.hidden_dim
        p += self.prism.num_iterations * 3 * self.hidden_dim * self.head_dim
        p += self.hidden_dim * self.intermediate_dim * 2
        p += self.hidden_dim * 2
        return p

    def count_parameters(self) -> int:
        total = self.vocab_size * self.hidden_dim
        total += self.count_layer_parameters() * self.num_layers
        if not self.tie_embeddings:
            total += self.vocab_size * self.hidden_dim
        return total + self.hidden_dim

    def estimate_memory(self) -> int:
        """Bytes per GPU by the reference's formula (config.zig:220-230): bf16 params +
        bf16 grads + 2x optimizer + activations for min(max_seq_len, 100k) tokens, all / 8."""
        pb = self.count_parameters() * 2
        act = min(self.max_seq_len, 100000) * self.hidden_dim * self.num_layers * 4
        return (pb + pb + 2 * pb + act) // 8


@dataclass
class TrainingConfig:  # config.zig:356-464
    total_steps: int = 1000000
    warmup_steps: int = 2000
    micro_batch_size: int = 1
    global_batch_size: int = 512
    gradient_accumulation_steps: int = 64
    learning_rate: float = 1e-4
    min_learning_rate: float = 1e-5
    weight_decay: float = 0.1
    gradient_clip: float = 1.0
    label_smoothing: float = 0.0
    optimizer: str = "lion_muon"
    lion_beta1: float = 0.95
    lion_beta2: float = 0.98
    muon_momentum: float = 0.95
    muon_iterations: int = 5
    lr_schedule: str = "cosine"
    mixed_precision: bool = True
    fp8_training: bool = True
    loss_scale: float = 65536.0
    dynamic_loss_scale: bool = True
    # extensions
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    fp8_gradients: bool = False  # with fp8_training: data / weight gradients on 8-bit operands too

    def validate(self) -> None:
        _enum(self.optimizer, OPTIMIZERS, "training.optimizer")
        _enum(self.lr_schedule, LR_SCHEDULES, "training.lr_schedule")
        if self.micro_batch_size <= 0:
            raise ConfigError("training.micro_batch_size must be positive")
        if self.gradient_accumulation_steps == 0:
            raise ConfigError("training.gradient_accumulation_steps must not be 0")
        if self.global_batch_size % self.micro_batch_size != 0:
            raise ConfigError("training.global_batch_size must be a multiple of micro_batch_size")


@dataclass
class RuntimeConfig:  # config.zig:481-538
    world_size: int = 8
    rank: int = 0
    tensor_parallel_size: int = 8
    pipeline_parallel_size: int = 1
    zero_stage: int = 2
    cpu_offload: bool = False
    nvme_offload: bool = False
    nvme_path: str = "/tmp/offload"
    seed: int = 42
    deterministic: bool = True
    # extensions
    context_parallel_size: int = 1
    data_parallel_size: int = 0

    def dp_size(self) -> int:
        if self.data_parallel_size > 0:
            return self.data_parallel_size
        denom = self.tensor_parallel_size * self.pipeline_parallel_size * self.context_parallel_size
        return max(1, self.world_size // max(1, denom))

    def validate(self) -> None:
        prod = (self.tensor_parallel_size * self.pipeline_parallel_size *
                self.context_parallel_size * self.dp_size())
        if prod != self.world_size:
            raise ConfigError(f"runtime: tp*pp*cp*dp = {prod} does not equal world_size "
                              f"{self.world_size}")
        if self.zero_stage not in (0, 1, 2, 3):
            raise ConfigError("runtime.zero_stage must be 0..3")


@dataclass
class SyntheticConfig:
    kind: str = ""  # "", "uniform" or "zipf"
    s: float = 1.1
    seed: int = 0


@dataclass
class DataConfig:  # config.zig:541-587
    path: str = "data/train.bin"
    tokenizer_path: str = "tokenizer.bin"
    seq_len: int = 8192
    shuffle_buffer_size: int = 10000
    prefetch_factor: int = 2
    num_workers: int = 4
    pack_sequences: bool = True
    # extension: the end-of-document token that pack_sequences cuts the stream at (the
    # tokenizer's <eos> is 259); -1 = the stream has no document marks, nothing to pack
    eos_token_id: int = -1
    synthetic: SyntheticConfig = field(default_factory=SyntheticConfig)


@dataclass
class CheckpointConfig:  # config.zig:590-631
    dir: str = "checkpoints"
    save_interval: int = 1000
    keep_last_n: int = 5
    save_optimizer: bool = True
    compression: bool = True
    async_save: bool = True


@dataclass
class TelemetryConfig:  # config.zig:634-676
    log_level: str = "info"
    log_file: str = "training.log"
    metrics_interval: int = 10
    enable_prometheus: bool = False
    prometheus_port: int = 9090
    track_memory: bool = True
    track_throughput: bool = True


SECTIONS = ("model", "training", "runtime", "data", "checkpoint", "telemetry")


@dataclass
class Config:  # config.zig:4-59
    model: ModelConfig = field(default_factory=ModelConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)
    data: DataConfig = field(default_factory=DataConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    telemetry: TelemetryConfig = field(default_factory=TelemetryConfig)

    @classmethod
    def from_dict(cls, d: dict, require_sections: bool = True) -> "Config":
        if not isinstance(d, dict):
            raise ConfigError("config root must be a map")
        if require_sections:
            for s in SECTIONS:
                if s not in d:
                    raise ConfigError(f"missing config section '{s}'")
        cfg = cls(
            model=_from_map(ModelConfig, d.get("model"), "model"),
            training=_from_map(TrainingConfig, d.get("training"), "training"),
            runtime=_from_map(RuntimeConfig, d.get("runtime"), "runtime"),
            data=_from_map(DataConfig, d.get("data"), "data"),
            checkpoint=_from_map(CheckpointConfig, d.get("checkpoint"), "checkpoint"),
            telemetry=_from_map(TelemetryConfig, d.get("telemetry"), "telemetry"),
        )
        _enum(cfg.telemetry.log_level, LOG_LEVELS, "telemetry.log_level")
        return cfg

    @classmethod
    def from_yaml(cls, text: str) -> "Config":
        return cls.from_dict(yaml_compat.loads(text))

    @classmethod
    def parse_from_file(cls, path) -> "Config":
        return cls.from_dict(yaml_compat.load(path))

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def to_yaml(self) -> str:
        return yaml_compat.dumps(self.to_dict()) + "\n"

    def config_hash(self) -> bytes:
        """32-byte digest stored in checkpoint metadata."""
        return hashlib.sha256(self.to_yaml().encode()).digest()

    def validate(self) -> list[str]:
        warns = self.model.validate()
        self.training.validate()
        self.runtime.validate()
        return warns


def parse_dtype(s: str):
    """config.zig:233-239"""
    import torch
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16,
            "fp8": torch.float8_e4m3fn}[_enum(s, DTYPES, "dtype")]
