"""Compiled-executor protocol, cache key and the compiled-plan wrapper.

Parity: ccdl_comm/executor.py:14-99.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, runtime_checkable

from ..config import CompressionConfig
from .info import ExecutionInfo
from .plan import WorkspacePolicy
from .work import CollectiveWork


@runtime_checkable
class CompiledExecutor(Protocol):
    execution_info: ExecutionInfo

    def run(self, tensor: object) -> CollectiveWork[object]: ...


class ObjectIdentity:
    """Hashes an arbitrary object by identity and keeps it alive."""

    __slots__ = ("_value",)

    def __init__(self, value: object | None) -> None:
        self._value = value

    @property
    def value(self) -> object | None:
        return self._value

    def __hash__(self) -> int:
        return id(self._value)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, ObjectIdentity) and other._value is self._value

    def __repr__(self) -> str:
        return f"ObjectIdentity(0x{id(self._value):x})"


@dataclass(frozen=True)
class CompileCacheKey:
    """Everything that can change what `backend.compile` produces."""

    registry_identity: ObjectIdentity
    backend: str
    collective: str
    requested_strategy: str
    executed_strategy: str
    fallback: tuple[str, ...]
    output_layout: str
    async_op: bool
    root: int
    reduce_op: str
    stage_signature: tuple[tuple[object, ...], ...]
    shape_class: tuple[int, ...]
    dtype: str
    layout: str
    rank: int
    world_size: int
    device: str
    local_rank: int | None
    local_world_size: int | None
    node_id: int | None
    node_count: int | None
    process_group_identity: ObjectIdentity
    process_group_identities: tuple[tuple[str, ObjectIdentity], ...]
    bit: int | None
    group_size: int | None
    compression: CompressionConfig | None
    topology_signature: str
    device_architecture: str
    strategy_policy_id: str | None
    workspace_budget_bytes: int | None
    allow_dynamic_shape: bool
    workspace_policy: WorkspacePolicy


@dataclass(frozen=True)
class CompiledCommunicationPlan:
    """A ready-to-run executor plus the facts it was compiled from."""

    executor: CompiledExecutor
    execution_info: ExecutionInfo
    cache_key: CompileCacheKey

    def run(self, tensor: object, *, out: object | None = None) -> CollectiveWork[object]:
        if out is None:
            return self.executor.run(tensor)
        key = self.cache_key
        if (key.collective, key.output_layout) != ("reduce_scatter", "shard"):
            raise TypeError("caller-owned shard output is supported only by reduce_scatter shard plans")
        return self.executor.run(tensor, out=out)
