"""Rank-local reduced shard plus the metadata a sharded optimizer needs.

Parity: ccdl_comm/shard.py:11-97 (same fields, invariants and derived values).
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any

from ._checks import need_shape


@dataclass(frozen=True)
class ReducedShard:
    shard: Any
    shard_index: int
    shard_numel: int
    original_shape: tuple[int, ...]
    original_numel: int
    world_size: int
    reduce: str
    padded_numel: int | None = None
    dtype: str = "auto"
    layout: str = "flat_contiguous"
    transport: str = "unknown"
    metadata: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.world_size <= 0:
            raise ValueError("world_size must be > 0")
        if self.shard_index < 0:
            raise ValueError("shard_index must be >= 0")
        if self.shard_index >= self.world_size:
            raise ValueError("shard_index must be < world_size")
        if self.shard_numel < 0:
            raise ValueError("shard_numel must be >= 0")
        if self.original_numel < 0:
            raise ValueError("original_numel must be >= 0")
        object.__setattr__(self, "original_shape", need_shape(self.original_shape, "original_shape"))
        span = self.shard_numel * self.world_size
        padded = span if self.padded_numel is None else self.padded_numel
        if padded < self.original_numel:
            raise ValueError("padded_numel must be >= original_numel")
        if padded != span:
            raise ValueError("padded_numel must equal shard_numel * world_size")
        object.__setattr__(self, "padded_numel", padded)
        object.__setattr__(self, "metadata", MappingProxyType(dict(self.metadata)))

    # Where the shard sits inside the flattened, unpadded tensor.
    @property
    def shard_offset(self) -> int:
        return self.shard_index * self.shard_numel

    @property
    def shard_end(self) -> int:
        return min(self.shard_offset + self.shard_numel, self.original_numel)

    @property
    def valid_numel(self) -> int:
        return max(0, self.shard_end - self.shard_offset)

    @property
    def padding_numel(self) -> int:
        return self.shard_numel - self.valid_numel

    @property
    def logical_range(self) -> tuple[int, int]:
        return (self.shard_offset, self.shard_end)

    @property
    def has_padding(self) -> bool:
        return self.padding_numel > 0 or int(self.padded_numel or 0) > self.original_numel

    @property
    def is_padding_only(self) -> bool:
        return self.valid_numel == 0

    def to_metadata(self) -> dict[str, Any]:
        keys = ("shard_index", "shard_numel", "shard_offset", "shard_end", "valid_numel",
                "original_shape", "original_numel", "padded_numel", "world_size", "reduce",
                "dtype", "layout", "transport")
        out = {k: getattr(self, k) for k in keys}
        out["metadata"] = dict(self.metadata)
        return out
