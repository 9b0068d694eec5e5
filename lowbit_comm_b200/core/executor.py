"""What `compile()` returns, and the key it is cached under.

A compiled plan is an executor (anything with `execution_info` and `run`) bound to the facts it was compiled
from.  Those facts form the cache key.  They are kept in three groups, which is also how a cache miss is
explained (`CompileCacheKey.differs_from`):

* `PlanFacts`      what was asked for and what was resolved (strategies, fallback chain, stages, compression)
* `TensorFacts`    what the tensor looks like (shape class, dtype, layout, workspace budget)
* `PlacementFacts` where this rank sits (rank, world, device, node layout, process groups by identity)

Every field is also readable directly on the key (`key.collective`, `key.bit`, `key.process_group_identity`
...), which keeps code written against the reference's flat key working (ccdl_comm/executor.py:44-81).
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Protocol, runtime_checkable

from ..config import CompressionConfig
from .info import ExecutionInfo
from .plan import CommunicationPlan, CompileContext, WorkspacePolicy
from .work import CollectiveWork


@runtime_checkable
class CompiledExecutor(Protocol):
    """The data-path object a backend hands back: no planning happens behind `run`."""

    execution_info: ExecutionInfo

    def run(self, tensor: object) -> CollectiveWork[object]: ...


class ObjectIdentity:
    """Wraps any object (a registry, a process group, None) so that it hashes and compares by identity.
    Holding the object keeps its id from being recycled while the key is alive."""

    __slots__ = ("_held",)

    def __init__(self, value: object | None) -> None:
        self._held = value

    @property
    def value(self) -> object | None:
        return self._held

    def __eq__(self, other: object) -> bool:
        return isinstance(other, ObjectIdentity) and other._held is self._held

    def __hash__(self) -> int:
        return hash(id(self._held))

    def __repr__(self) -> str:
        return f"ObjectIdentity({type(self._held).__name__} at 0x{id(self._held):x})"


def _stage_facts(stage: Any) -> tuple[object, ...]:
    return (stage.name, stage.collective, stage.strategy, stage.backend, stage.compression,
            ObjectIdentity(stage.process_group), stage.output_layout, stage.async_op)


@dataclass(frozen=True)
class PlanFacts:
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
    compression: CompressionConfig | None
    workspace_policy: WorkspacePolicy
    strategy_policy_id: str | None

    @property
    def bit(self) -> int | None:
        return None if self.compression is None else self.compression.bit

    @property
    def group_size(self) -> int | None:
        return None if self.compression is None else self.compression.group_size


@dataclass(frozen=True)
class TensorFacts:
    shape_class: tuple[int, ...]
    dtype: str
    layout: str
    workspace_budget_bytes: int | None
    allow_dynamic_shape: bool


@dataclass(frozen=True)
class PlacementFacts:
    rank: int
    world_size: int
    device: str
    local_rank: int | None
    local_world_size: int | None
    node_id: int | None
    node_count: int | None
    process_group_identity: ObjectIdentity
    process_group_identities: tuple[tuple[str, ObjectIdentity], ...]
    topology_signature: str
    device_architecture: str


@dataclass(frozen=True)
class CompileCacheKey:
    """Everything that can change what `backend.compile` produces, grouped."""

    registry_identity: ObjectIdentity
    plan: PlanFacts
    tensor: TensorFacts
    placement: PlacementFacts

    @classmethod
    def of(cls, requested: CommunicationPlan, effective: CommunicationPlan, context: CompileContext,
           registry: object, strategy_policy_id: str | None) -> "CompileCacheKey":
        """Key of compiling `effective` (what `requested` resolved to) for `context` with `registry`.
        Shapes are exact: no backend proves a wider shape class yet."""

        plan = PlanFacts(
            backend=effective.backend, collective=effective.collective, requested_strategy=requested.strategy,
            executed_strategy=effective.strategy, fallback=requested.fallback, output_layout=effective.output_layout,
            async_op=effective.async_op, root=effective.root, reduce_op=effective.reduce_op,
            stage_signature=tuple(_stage_facts(s) for s in effective.stages), compression=effective.compression,
            workspace_policy=effective.workspace_policy, strategy_policy_id=strategy_policy_id)
        tensor = TensorFacts(context.shape, context.dtype, context.layout, context.workspace_budget_bytes,
                             context.allow_dynamic_shape)
        groups = tuple((name, ObjectIdentity(group)) for name, group in sorted(context.process_groups.items()))
        placement = PlacementFacts(
            rank=context.rank, world_size=context.world_size, device=context.device, local_rank=context.local_rank,
            local_world_size=context.local_world_size, node_id=context.node_id, node_count=context.node_count,
            process_group_identity=ObjectIdentity(context.process_group), process_group_identities=groups,
            topology_signature=context.topology_signature, device_architecture=context.device_architecture)
        return cls(ObjectIdentity(registry), plan, tensor, placement)

    def __getattr__(self, name: str) -> Any:
        # flat access to the grouped facts; only reached for names that are not fields of the key itself
        if name.startswith("__"):
            raise AttributeError(name)
        for part in ("plan", "tensor", "placement"):
            group = object.__getattribute__(self, part)
            if name in {f.name for f in fields(group)} or isinstance(getattr(type(group), name, None), property):
                return getattr(group, name)
        raise AttributeError(f"{type(self).__name__!s} has no fact named {name!r}")

    def differs_from(self, other: "CompileCacheKey") -> tuple[str, ...]:
        """Names of the facts in which two keys differ (why a lookup missed)."""

        changed = [] if self.registry_identity == other.registry_identity else ["registry_identity"]
        for part in ("plan", "tensor", "placement"):
            mine, theirs = getattr(self, part), getattr(other, part)
            changed += [f.name for f in fields(mine) if getattr(mine, f.name) != getattr(theirs, f.name)]
        return tuple(changed)


@dataclass(frozen=True)
class CompiledCommunicationPlan:
    """A ready-to-run executor plus the facts it was compiled from."""

    executor: CompiledExecutor
    execution_info: ExecutionInfo
    cache_key: CompileCacheKey

    def run(self, tensor: object, *, out: object | None = None) -> CollectiveWork[object]:
        if out is not None:
            produces_shard = (self.cache_key.collective, self.cache_key.output_layout) == ("reduce_scatter", "shard")
            if not produces_shard:
                raise TypeError("`out=` names a caller-owned shard buffer; only reduce_scatter plans with shard "
                                "output accept it")
            return self.executor.run(tensor, out=out)
        return self.executor.run(tensor)
