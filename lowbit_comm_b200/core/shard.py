"""The result of a compressed reduce-scatter: this rank's reduced shard and where it belongs.

A sharded optimizer (ZeRO / FSDP style) consumes `shard` together with the geometry: which slice of the
flattened gradient it is, how much of it is padding, and how the tensor was split.  The constructor arguments
and the derived names follow the reference (ccdl_comm/shard.py:11-97) so that consumers written against it keep
working; the geometry itself is computed once into a `ShardSpan`.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, NamedTuple

from ._checks import need_shape


class ShardSpan(NamedTuple):
    """Half-open element range [offset, end) of a shard inside the flattened, unpadded tensor, and its padding."""

    offset: int
    end: int
    padding: int

    @property
    def valid(self) -> int:
        return max(0, self.end - self.offset)

    @classmethod
    def locate(cls, index: int, shard_numel: int, original_numel: int) -> "ShardSpan":
        offset = index * shard_numel
        end = min(offset + shard_numel, original_numel)
        return cls(offset, end, shard_numel - max(0, end - offset))


_NON_NEGATIVE = ("shard_index", "shard_numel", "original_numel")
_DESCRIBED = ("shard_index", "shard_numel", "shard_offset", "shard_end", "valid_numel", "original_shape",
              "original_numel", "padded_numel", "world_size", "reduce", "dtype", "layout", "transport")


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
        for name in _NON_NEGATIVE:
            if getattr(self, name) < 0:
                raise ValueError(f"{name} must be >= 0")
        if self.shard_index >= self.world_size:
            raise ValueError("shard_index must be < world_size")
        whole = self.shard_numel * self.world_size          # the padded tensor is W equal shards, nothing else
        padded = whole if self.padded_numel is None else self.padded_numel
        if padded < self.original_numel:
            raise ValueError("padded_numel must be >= original_numel")
        if padded != whole:
            raise ValueError("padded_numel must equal shard_numel * world_size")
        frozen = {"original_shape": need_shape(self.original_shape, "original_shape"), "padded_numel": padded,
                  "metadata": MappingProxyType(dict(self.metadata))}
        for name, value in frozen.items():
            object.__setattr__(self, name, value)

    # -- geometry ---------------------------------------------------------------------------------
    @property
    def span(self) -> ShardSpan:
        return ShardSpan.locate(self.shard_index, self.shard_numel, self.original_numel)

    shard_offset = property(lambda self: self.span.offset)
    shard_end = property(lambda self: self.span.end)
    valid_numel = property(lambda self: self.span.valid)
    padding_numel = property(lambda self: self.span.padding)
    logical_range = property(lambda self: (self.span.offset, self.span.end))

    @property
    def has_padding(self) -> bool:
        """Padding in this shard, or anywhere in the padded tensor."""

        return self.span.padding > 0 or (self.padded_numel or 0) > self.original_numel

    @property
    def is_padding_only(self) -> bool:
        return self.span.valid == 0

    def valid_view(self) -> Any:
        """The part of `shard` that holds real elements (a view when `shard` supports slicing)."""

        return self.shard[: self.span.valid]

    def to_metadata(self) -> dict[str, Any]:
        """Everything except the tensor, as plain values (for logs and for `all_gather_object` checks)."""

        described = {name: getattr(self, name) for name in _DESCRIBED}
        described["metadata"] = dict(self.metadata)
        return described
