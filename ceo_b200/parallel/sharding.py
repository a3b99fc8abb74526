"""Shard arithmetic and the parallel layout description, and the device mesh built from it.

Counterpart of src/tensor/sharding.zig: ``ShardSpec.local_shape / global_offset`` with the
remainder going to the first shards (sharding.zig:90-181), ``TensorParallelConfig`` with the
shard dimension of each layer kind (183-222), ``SequenceParallelConfig`` (224-287),
``ZeroConfig`` with 1 MiB-chunk round-robin ownership (289-355), ``ParallelConfig`` and its
rank ordering pp -> dp -> tp -> sp innermost (357-421), ``ShardedTensor`` (424-457).
The reference never consults these; here ``DeviceMesh`` turns a ``ParallelConfig`` into
``torch.distributed`` groups that the FSDP / TP / CP code uses.
"""
from __future__ import annotations

from dataclasses import dataclass, field

ZERO_CHUNK_BYTES = 1 << 20


class ParallelError(ValueError):
    pass


@dataclass(frozen=True)
class ShardSpec:
    shard_dim: int | None  # None = not sharded
    num_shards: int = 1
    shard_idx: int = 0

    def __post_init__(self):
        if self.num_shards <= 0:
            raise ParallelError("num_shards must be positive")
        if not 0 <= self.shard_idx < self.num_shards:
            raise ParallelError("shard_idx out of range")
        if self.shard_dim is None and self.num_shards != 1:
            raise ParallelError("an unsharded spec has exactly one shard")

    @classmethod
    def no_sharding(cls):
        return cls(None, 1, 0)

    @property
    def is_first(self):
        return self.shard_idx == 0

    @property
    def is_last(self):
        return self.shard_idx == self.num_shards - 1

    def _split(self, size: int):
        base, rem = divmod(size, self.num_shards)
        if self.shard_idx < rem:
            return base + 1, self.shard_idx * (base + 1)
        return base, rem * (base + 1) + (self.shard_idx - rem) * base

    def local_shape(self, global_shape) -> tuple:
        shape = tuple(global_shape)
        if self.shard_dim is None:
            return shape
        if not shape:
            raise ParallelError("cannot shard a scalar")
        if not 0 <= self.shard_dim < len(shape):
            raise ParallelError("shard dimension outside the tensor rank")
        loc, _ = self._split(shape[self.shard_dim])
        return shape[:self.shard_dim] + (loc,) + shape[self.shard_dim + 1:]

    def global_offset(self, global_shape) -> tuple:
        shape = tuple(global_shape)
        off = [0] * len(shape)
        if self.shard_dim is None:
            return tuple(off)
        if not 0 <= self.shard_dim < len(shape):
            raise ParallelError("shard dimension outside the tensor rank")
        _, o = self._split(shape[self.shard_dim])
        off[self.shard_dim] = o
        return tuple(off)

    def slice_of(self, tensor):
        """The local shard of a full tensor (a view)."""
        if self.shard_dim is None:
            return tensor
        n, o = self._split(tensor.shape[self.shard_dim])
        return tensor.narrow(self.shard_dim, o, n)


@dataclass
class TensorParallelConfig:
    """Which dimension of each (out, in)-oriented weight is split (sharding.zig:183-222):
    column-parallel layers split the output features, row-parallel layers the input."""
    world_size: int = 1
    rank: int = 0
    embed_dim: int = 0      # vocabulary rows
    qkv_dim: int = 0        # output features (heads)
    attn_out_dim: int = 1   # input features
    mlp_up_dim: int = 0
    mlp_down_dim: int = 1

    def spec(self, kind: str) -> ShardSpec:
        if self.world_size == 1:
            return ShardSpec.no_sharding()
        d = {"embed": self.embed_dim, "qkv": self.qkv_dim, "attn_out": self.attn_out_dim,
             "mlp_up": self.mlp_up_dim, "mlp_down": self.mlp_down_dim}[kind]
        return ShardSpec(d, self.world_size, self.rank)


@dataclass
class SequenceParallelConfig:
    world_size: int = 1
    rank: int = 0
    seq_dim: int = 1
    use_ring_attention: bool = False  # the reference's flag; EFLA needs a state prefix instead

    def local_seq_len(self, seq_len: int) -> int:
        return ShardSpec(0, self.world_size, self.rank).local_shape((seq_len,))[0]

    def seq_offset(self, seq_len: int) -> int:
        return ShardSpec(0, self.world_size, self.rank).global_offset((seq_len,))[0]


@dataclass
class ZeroConfig:
    stage: int = 0
    offload_optimizer: bool = False
    offload_params: bool = False
    partition_optimizer: bool = True
    partition_gradients: bool = True
    partition_params: bool = False

    @classmethod
    def for_stage(cls, stage: int) -> "ZeroConfig":
        if stage not in (0, 1, 2, 3):
            raise ParallelError("zero stage must be 0..3")
        return cls(stage, partition_optimizer=stage >= 1, partition_gradients=stage >= 2,
                   partition_params=stage >= 3)

    def owns_parameter(self, byte_offset: int, rank: int, world: int) -> bool:
        """1 MiB chunks dealt round-robin (sharding.zig:340-355)."""
        if self.stage == 0 or world <= 1:
            return True
        return (byte_offset // ZERO_CHUNK_BYTES) % world == rank


@dataclass
class ParallelConfig:
    pp_world_size: int = 1
    pp_rank: int = 0
    dp_world_size: int = 1
    dp_rank: int = 0
    tp_world_size: int = 1
    tp_rank: int = 0
    sp_world_size: int = 1   # innermost axis: sequence / context parallel
    sp_rank: int = 0
    zero: ZeroConfig = field(default_factory=ZeroConfig)

    def global_rank(self) -> int:
        r = self.pp_rank
        r = r * self.dp_world_size + self.dp_rank
        r = r * self.tp_world_size + self.tp_rank
        return r * self.sp_world_size + self.sp_rank

    def global_world_size(self) -> int:
        return self.pp_world_size * self.dp_world_size * self.tp_world_size * self.sp_world_size

    @classmethod
    def from_global_rank(cls, rank: int, pp: int, dp: int, tp: int, sp: int = 1,
                         zero_stage: int = 0) -> "ParallelConfig":
        if not 0 <= rank < pp * dp * tp * sp:
            raise ParallelError("rank outside the mesh")
        sp_r = rank % sp
        rank //= sp
        tp_r = rank % tp
        rank //= tp
        dp_r = rank % dp
        pp_r = rank // dp
        return cls(pp, pp_r, dp, dp_r, tp, tp_r, sp, sp_r, ZeroConfig.for_stage(zero_stage))

    @classmethod
    def from_runtime(cls, rt, rank: int) -> "ParallelConfig":
        """From a ``RuntimeConfig`` (utils/config.py)."""
        return cls.from_global_rank(rank, rt.pipeline_parallel_size, rt.dp_size(),
                                    rt.tensor_parallel_size, rt.context_parallel_size,
                                    rt.zero_stage)

    def group_ranks(self, axis: str) -> list[int]:
        """Global ranks of the group this rank belongs to along ``axis`` (pp|dp|tp|sp)."""
        out = []
        sizes = {"pp": self.pp_world_size, "dp": self.dp_world_size, "tp": self.tp_world_size,
                 "sp": self.sp_world_size}
        for i in range(sizes[axis]):
            c = ParallelConfig(self.pp_world_size, self.pp_rank, self.dp_world_size, self.dp_rank,
                               self.tp_world_size, self.tp_rank, self.sp_world_size, self.sp_rank)
            setattr(c, axis + "_rank", i)
            out.append(c.global_rank())
        return out


@dataclass
class ShardedTensor:
    local: object
    spec: ShardSpec
    global_shape: tuple

    def global_offset(self):
        return self.spec.global_offset(self.global_shape)


class DeviceMesh:
    """Process groups for every axis of a ``ParallelConfig`` (all ranks must construct it,
    in the same order, because ``new_group`` is collective)."""

    def __init__(self, pc: ParallelConfig):
        import torch.distributed as dist
        self.pc = pc
        self.groups = {}
        world = pc.global_world_size()
        if not dist.is_initialized() or world == 1:
            return
        for axis in ("pp", "dp", "tp", "sp"):
            seen = set()
            for r in range(world):
                c = ParallelConfig.from_global_rank(r, pc.pp_world_size, pc.dp_world_size,
                                                    pc.tp_world_size, pc.sp_world_size)
                ranks = tuple(c.group_ranks(axis))
                if ranks in seen:
                    continue
                seen.add(ranks)
                g = dist.new_group(list(ranks)) if len(ranks) > 1 else None
                if pc.global_rank() in ranks:
                    self.groups[axis] = g

    def group(self, axis: str):
        return self.groups.get(axis)
