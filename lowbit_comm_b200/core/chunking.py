"""Equal-shard chunk plans.

`ChunkPlan` mirrors the reference's element-granular plan
(ccdl_comm/cuda/transports/compressed_reduce_scatter.py:8-94: shard = ceil(n/W),
rank r owns chunk r).  `GroupShardPlan` is the plan the fused sm_100a kernels
use: shards are counted in quantization groups and rounded up to a multiple of
`align_groups` so every shard's value and scale regions start on a 16-byte
boundary inside a planar payload.
"""

from __future__ import annotations

from dataclasses import dataclass


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass(frozen=True)
class ChunkRange:
    """Half-open range of the flattened (padded) tensor owned by one destination rank."""

    start: int
    stop: int

    def __post_init__(self) -> None:
        for value, name in ((self.start, "chunk start"), (self.stop, "chunk stop")):
            if isinstance(value, bool) or not isinstance(value, int):
                raise TypeError(f"{name} must be an integer")
        if self.start < 0:
            raise ValueError("chunk start must be >= 0")
        if self.stop < self.start:
            raise ValueError("chunk stop must be >= start")

    @property
    def numel(self) -> int:
        return self.stop - self.start


@dataclass(frozen=True)
class ChunkPlan:
    numel: int
    world_size: int
    shard_numel: int
    padded_numel: int

    @classmethod
    def build(cls, numel: int, world_size: int) -> "ChunkPlan":
        if numel < 0:
            raise ValueError("numel must be >= 0")
        if world_size <= 0:
            raise ValueError("world_size must be > 0")
        shard = _ceil_div(numel, world_size) if numel else 0
        return cls(numel, world_size, shard, shard * world_size)

    @property
    def padding_numel(self) -> int:
        return self.padded_numel - self.numel

    def owner(self, chunk: int) -> int:
        self._check(chunk)
        return chunk

    def bounds(self, chunk: int) -> tuple[int, int]:
        """Half-open element range of `chunk` inside the padded tensor."""

        self._check(chunk)
        return chunk * self.shard_numel, (chunk + 1) * self.shard_numel

    def valid_bounds(self, chunk: int) -> tuple[int, int]:
        lo, hi = self.bounds(chunk)
        return min(lo, self.numel), min(hi, self.numel)

    def _check(self, chunk: int) -> None:
        if not 0 <= chunk < self.world_size:
            raise ValueError("chunk index out of range")

    # the reference's field names (compressed_reduce_scatter.py:28-69)
    @property
    def original_numel(self) -> int:
        return self.numel

    @property
    def chunks(self) -> tuple[ChunkRange, ...]:
        return tuple(ChunkRange(*self.bounds(c)) for c in range(self.world_size))

    @property
    def owner_by_chunk(self) -> tuple[int, ...]:
        return tuple(range(self.world_size))

    def chunk_for_rank(self, rank: int) -> ChunkRange:
        if isinstance(rank, bool) or not isinstance(rank, int):
            raise TypeError("rank must be an integer")
        if not 0 <= rank < self.world_size:
            raise ValueError(f"rank must be in [0, {self.world_size})")
        return ChunkRange(*self.bounds(rank))


def compile_chunk_plan(*, original_numel: int, world_size: int) -> ChunkPlan:
    """The reference's constructor name for `ChunkPlan.build`."""

    for value, name in ((original_numel, "original_numel"), (world_size, "world_size")):
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError(f"{name} must be an integer")
    return ChunkPlan.build(original_numel, world_size)


@dataclass(frozen=True)
class GroupShardPlan:
    """Shard plan in units of quantization groups (fused-kernel layout)."""

    numel: int
    world_size: int
    group_size: int
    align_groups: int
    num_groups: int          # groups that hold real data: ceil(numel / group_size)
    shard_groups: int        # groups per rank (multiple of align_groups)

    @classmethod
    def build(cls, numel: int, world_size: int, group_size: int, align_groups: int = 8) -> "GroupShardPlan":
        if numel < 0 or world_size <= 0 or group_size <= 0 or align_groups <= 0:
            raise ValueError("invalid shard plan arguments")
        groups = _ceil_div(numel, group_size)
        per_rank = _ceil_div(groups, world_size)
        per_rank = _ceil_div(per_rank, align_groups) * align_groups if per_rank else 0
        return cls(numel, world_size, group_size, align_groups, groups, per_rank)

    @property
    def total_groups(self) -> int:
        return self.shard_groups * self.world_size

    @property
    def shard_numel(self) -> int:
        return self.shard_groups * self.group_size

    @property
    def padded_numel(self) -> int:
        return self.shard_numel * self.world_size

    def shard_valid_numel(self, rank: int) -> int:
        lo = rank * self.shard_numel
        return max(0, min(self.numel, lo + self.shard_numel) - lo)

    def shard_valid_groups(self, rank: int) -> int:
        lo = rank * self.shard_groups
        return max(0, min(self.num_groups, lo + self.shard_groups) - lo)


def hierarchy_groups(ranks: list[int] | tuple[int, ...], local_group_size: int) -> tuple[list[list[int]], list[list[int]]]:
    """Contiguous two-level grouping of `ranks` (global ranks of one process group, in group order).

    Returns (local groups, inter groups): `len(ranks) / L` local groups of L consecutive ranks, and L inter
    groups that hold the ranks with the same position in every local group.  Rank r sits in local group
    r // L with local rank r % L, and in inter group r % L with inter rank r // L.  This is the membership
    rule of the reference's hierarchical stages (ccdl_comm/communication/hierarchical_transport.py:178-215;
    cuda/transports/hierarchical.py:184-265), e.g. 8 ranks as 2 x 4: full -> 4-rank shard -> 2-rank
    all-reduce of the shard -> 4-rank restore.
    """

    L = int(local_group_size)
    world = len(ranks)
    if L <= 0 or world == 0 or world % L != 0:
        raise ValueError(f"{world} ranks cannot be split into local groups of {L}")
    nodes = world // L
    local = [[ranks[node * L + i] for i in range(L)] for node in range(nodes)]
    inter = [[ranks[node * L + lane] for node in range(nodes)] for lane in range(L)]
    return local, inter
