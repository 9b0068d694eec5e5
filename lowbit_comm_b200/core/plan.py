"""Immutable communication requests and the static facts they compile against.

Parity: ccdl_comm/plan.py:13-129 and ccdl_comm/stage.py:15-32.  Nothing in this
module imports torch; process groups are carried as opaque objects.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field

from ..config import CompressionConfig
from ._checks import (freeze, is_plain_int, need_optional_index, need_optional_minimum, need_shape, need_texts,
                      read_only, text_tuple)

_DTYPE_BYTES = {"fp16": 2, "bf16": 2, "fp32": 4, "float16": 2, "bfloat16": 2, "float32": 4}


def _check_compression(value) -> None:
    if value is not None and not isinstance(value, CompressionConfig):
        raise TypeError("compression must be a CompressionConfig or None")


@dataclass(frozen=True)
class CommunicationStage:
    """One step of a multi-stage (hierarchical) plan."""

    name: str
    collective: str
    strategy: str
    backend: str = "cuda"
    compression: CompressionConfig | None = None
    process_group: object | None = None
    output_layout: str = "full"
    async_op: bool = True

    def __post_init__(self) -> None:
        need_texts(self, "name", "collective", "strategy", "backend", "output_layout")
        _check_compression(self.compression)

    @property
    def key(self) -> tuple[str, str, str, str]:
        """(collective, strategy, backend, output layout): what a registry is asked for."""

        return (self.collective, self.strategy, self.backend, self.output_layout)


@dataclass(frozen=True)
class WorkspacePolicy:
    """Limits for workspace caching; owns no buffers itself."""

    cache: bool = True
    max_cached_bytes: int | None = None
    max_entries: int | None = None
    stream_safe: bool = True

    def __post_init__(self) -> None:
        need_optional_minimum(self.max_cached_bytes, 0, "max_cached_bytes")
        need_optional_minimum(self.max_entries, 1, "max_entries")

    def admits(self, cached_bytes: int, entries: int) -> bool:
        """Whether a cache holding `cached_bytes` in `entries` buffers is inside the policy."""

        if not self.cache:
            return cached_bytes == 0 and entries == 0
        return (self.max_cached_bytes is None or cached_bytes <= self.max_cached_bytes) and \
            (self.max_entries is None or entries <= self.max_entries)


@dataclass(frozen=True)
class CommunicationPlan:
    """What the caller wants: collective, strategy, compression, layout."""

    collective: str
    strategy: str
    backend: str = "cuda"
    compression: CompressionConfig | None = None
    stages: tuple[CommunicationStage, ...] = ()
    fallback: tuple[str, ...] = ()
    output_layout: str = "full"
    async_op: bool = True
    root: int = 0
    reduce_op: str = "mean"
    workspace_policy: WorkspacePolicy = WorkspacePolicy()

    def __post_init__(self) -> None:
        need_texts(self, "collective", "strategy", "backend", "output_layout", "reduce_op")
        _check_compression(self.compression)
        if not isinstance(self.workspace_policy, WorkspacePolicy):
            raise TypeError("workspace_policy must be a WorkspacePolicy")
        if not is_plain_int(self.root) or self.root < 0:
            raise ValueError("root must be a non-negative integer")
        stages = tuple(self.stages)
        if not all(isinstance(s, CommunicationStage) for s in stages):
            raise TypeError("stages must contain only CommunicationStage values")
        freeze(self, stages=stages,
               fallback=text_tuple(self.fallback, "fallback", message="fallback strategy must be a non-empty string"))
        if self.strategy == "hierarchical" and not stages:
            raise ValueError("hierarchical strategy requires at least one stage")

    @property
    def key(self) -> tuple[str, str, str, str]:
        return (self.collective, self.strategy, self.backend, self.output_layout)

    @property
    def is_compressed(self) -> bool:
        return self.compression is not None and self.strategy != "native_nccl"

    def candidates(self) -> tuple[str, ...]:
        """The requested strategy followed by its fallback chain, duplicates removed, in order."""

        return tuple(dict.fromkeys((self.strategy, *self.fallback)))


@dataclass(frozen=True)
class CompileContext:
    """Rank, tensor and topology facts known before the first launch."""

    rank: int
    world_size: int
    device: str
    shape: tuple[int, ...]
    dtype: str
    layout: str = "contiguous"
    local_rank: int | None = None
    local_world_size: int | None = None
    node_id: int | None = None
    node_count: int | None = None
    process_group: object | None = None
    process_groups: Mapping[str, object] = field(default_factory=dict)
    topology_signature: str = "unknown"
    workspace_budget_bytes: int | None = None
    allow_dynamic_shape: bool = False
    device_architecture: str = "unknown"

    def __post_init__(self) -> None:
        if self.world_size <= 0:
            raise ValueError("world_size must be > 0")
        if not 0 <= self.rank < self.world_size:
            raise ValueError("rank must be >= 0 and < world_size")
        need_texts(self, "device", "dtype", "layout", "topology_signature", "device_architecture")
        need_optional_minimum(self.local_world_size, 1, "local_world_size")
        need_optional_index(self.local_rank, self.local_world_size, "local_rank", "local_world_size")
        need_optional_minimum(self.node_count, 1, "node_count")
        need_optional_index(self.node_id, self.node_count, "node_id", "node_count")
        need_optional_minimum(self.workspace_budget_bytes, 0, "workspace_budget_bytes")
        groups = dict(self.process_groups)
        if any(not isinstance(k, str) or not k.strip() for k in groups):
            raise ValueError("process_groups keys must be non-empty strings")
        freeze(self, shape=need_shape(self.shape), process_groups=read_only(groups))

    @property
    def numel(self) -> int:
        total = 1
        for dim in self.shape:
            total *= dim
        return total

    @property
    def nbytes(self) -> int:
        """Bytes of the tensor when the dtype name is one of the source dtypes (fp16 / bf16 / fp32), else 0."""

        return self.numel * _DTYPE_BYTES.get(self.dtype, 0)

    @property
    def has_node_layout(self) -> bool:
        """True when local rank / local world size / node id / node count are all known and consistent."""

        facts = (self.local_rank, self.local_world_size, self.node_id, self.node_count)
        if any(f is None for f in facts):
            return False
        return self.world_size == self.local_world_size * self.node_count and \
            self.rank == self.node_id * self.local_world_size + self.local_rank
