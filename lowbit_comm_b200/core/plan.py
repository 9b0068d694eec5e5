"""Immutable communication requests and the static facts they compile against.

Parity: ccdl_comm/plan.py:13-129 and ccdl_comm/stage.py:15-32.  Nothing in this
module imports torch; process groups are carried as opaque objects.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field
from types import MappingProxyType

from ..config import CompressionConfig
from ._checks import is_plain_int, need_optional_index, need_shape, need_text


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
        for attr in ("name", "collective", "strategy", "backend", "output_layout"):
            need_text(getattr(self, attr), attr)
        _check_compression(self.compression)


@dataclass(frozen=True)
class WorkspacePolicy:
    """Limits for workspace caching; owns no buffers itself."""

    cache: bool = True
    max_cached_bytes: int | None = None
    max_entries: int | None = None
    stream_safe: bool = True

    def __post_init__(self) -> None:
        if self.max_cached_bytes is not None and self.max_cached_bytes < 0:
            raise ValueError("max_cached_bytes must be >= 0")
        if self.max_entries is not None and self.max_entries <= 0:
            raise ValueError("max_entries must be > 0")


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
        for attr in ("collective", "strategy", "backend", "output_layout"):
            need_text(getattr(self, attr), attr)
        need_text(self.reduce_op, "reduce_op")
        _check_compression(self.compression)
        if not isinstance(self.workspace_policy, WorkspacePolicy):
            raise TypeError("workspace_policy must be a WorkspacePolicy")
        if not is_plain_int(self.root) or self.root < 0:
            raise ValueError("root must be a non-negative integer")
        stages = tuple(self.stages)
        if not all(isinstance(s, CommunicationStage) for s in stages):
            raise TypeError("stages must contain only CommunicationStage values")
        fallback = tuple(self.fallback)
        for name in fallback:
            need_text(name, "fallback strategy")
        object.__setattr__(self, "stages", stages)
        object.__setattr__(self, "fallback", fallback)
        if self.strategy == "hierarchical" and not stages:
            raise ValueError("hierarchical strategy requires at least one stage")


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
        for attr in ("device", "dtype", "layout", "topology_signature", "device_architecture"):
            need_text(getattr(self, attr), attr)
        object.__setattr__(self, "shape", need_shape(self.shape))
        if self.local_world_size is not None and self.local_world_size <= 0:
            raise ValueError("local_world_size must be > 0")
        need_optional_index(self.local_rank, self.local_world_size, "local_rank", "local_world_size")
        if self.node_count is not None and self.node_count <= 0:
            raise ValueError("node_count must be > 0")
        need_optional_index(self.node_id, self.node_count, "node_id", "node_count")
        if self.workspace_budget_bytes is not None and self.workspace_budget_bytes < 0:
            raise ValueError("workspace_budget_bytes must be >= 0")
        groups = dict(self.process_groups)
        if any(not isinstance(k, str) or not k.strip() for k in groups):
            raise ValueError("process_groups keys must be non-empty strings")
        object.__setattr__(self, "process_groups", MappingProxyType(groups))

    @property
    def numel(self) -> int:
        total = 1
        for dim in self.shape:
            total *= dim
        return total
