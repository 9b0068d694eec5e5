"""Compile-once stage chains for the hierarchical all-reduce (torch-free).

A hierarchical plan is a `CommunicationPlan(strategy="hierarchical")` whose `stages` spell out the chain
full -> shard -> shard -> full:

    reduce_scatter  over the ranks of this node            (full  -> shard)
    all_reduce      over the ranks with my local index      (shard -> shard)
    all_gather      over the ranks of this node again       (shard -> full)

`compile_hierarchical_stages` checks the chain, works out which ranks take part in every stage from the
topology fields of the `CompileContext` (local rank / local world size / node id / node count), obtains
one process group per stage (given on the stage, given by name in `context.process_groups`, or created
by `group_factory`), verifies its members, and binds one operation per stage through `operation_factory`.
The result runs the chain without a host wait in between: a stage that has a stream makes that stream
wait for the previous stage's completion.

Role parity: ccdl_comm/cuda/transports/hierarchical.py:27-270 (`StageExecution`, `CompiledStage`,
`HierarchicalExecutor`, `compile_hierarchical_stages`).  On one NVSwitch node the "nodes" are groups of
GPUs (2 x 4 on eight); the CUDA backend binds the stages to the fused kernels of the sub-groups.
"""

from __future__ import annotations

import threading
from collections.abc import Callable, Sequence
from dataclasses import dataclass, replace
from typing import Any

from ..exceptions import UnsupportedCollective
from .plan import CommunicationPlan, CommunicationStage, CompileContext
from .work import CompletionWork

# (collective, layout in, layout out) -> which ranks take part
_TRANSITIONS = {
    ("reduce_scatter", "full", "shard"): "local",
    ("all_reduce", "shard", "shard"): "inter",
    ("all_gather", "shard", "full"): "local",
}
_INTER_STRATEGIES = frozenset({"topology", "all_gather", "reduce_scatter", "compressed", "auto", "native_nccl"})
_GATHER_STRATEGIES = frozenset({"native_nccl", "compressed", "all_gather"})


@dataclass(frozen=True)
class StageExecution:
    """What one launched stage produced, and the device-side event after which it is valid."""

    value: object
    completion: object | None = None
    resources: tuple[object, ...] = ()

    def __post_init__(self) -> None:
        object.__setattr__(self, "resources", tuple(self.resources))


@dataclass(frozen=True)
class CompiledStage:
    """A stage with its participants, layouts, process group, stream and operation bound."""

    name: str
    input_layout: str
    output_layout: str
    participants: tuple[int, ...]
    process_group: object
    operation: Callable[..., Any]
    stream: object | None = None
    completion_factory: Callable[[object | None], object] | None = None

    def __post_init__(self) -> None:
        if not self.name.strip():
            raise ValueError("compiled stage name must be non-empty")
        if not callable(self.operation):
            raise TypeError("stage operation must be callable")
        object.__setattr__(self, "participants", tuple(int(r) for r in self.participants))
        if not self.participants or len(set(self.participants)) != len(self.participants):
            raise ValueError("stage participants must be distinct ranks")

    def launch(self, value: object, dependency: object | None) -> StageExecution:
        """Order this stage after `dependency` (on the stream when there is one), then run the operation."""

        if dependency is not None:
            wait_stream = getattr(dependency, "wait_stream", None)
            if self.stream is not None and callable(wait_stream):
                wait_stream(self.stream)
            else:
                waiter = getattr(dependency, "wait", None)
                if callable(waiter):
                    waiter()
        produced = self.operation(value)
        if isinstance(produced, StageExecution):
            return produced
        completion = self.completion_factory(self.stream) if self.completion_factory is not None else None
        return StageExecution(produced, completion, (value,))

    def emergency_completion(self) -> object | None:
        """An event behind whatever the failed stage may have enqueued (None when there is no way to make one)."""

        if self.completion_factory is None:
            return None
        try:
            return self.completion_factory(self.stream)
        except Exception:  # noqa: BLE001 - already on an error path
            return None


class HierarchicalExecutor:
    """Runs an immutable stage chain; returns work bound to the last stage's completion."""

    def __init__(self, stages: Sequence[CompiledStage]) -> None:
        stages = tuple(stages)
        if not stages:
            raise ValueError("hierarchical executor requires at least one compiled stage")
        for before, after in zip(stages, stages[1:]):
            if before.output_layout != after.input_layout:
                raise ValueError(f"stage layout mismatch: {before.name!r} outputs {before.output_layout!r}, "
                                 f"but {after.name!r} consumes {after.input_layout!r}")
        self.stages = stages
        self._quarantine: list[tuple[tuple[object, ...], object | None]] = []
        self._lock = threading.Lock()

    @property
    def input_layout(self) -> str:
        return self.stages[0].input_layout

    @property
    def output_layout(self) -> str:
        return self.stages[-1].output_layout

    @property
    def pending_failure_count(self) -> int:
        with self._lock:
            return len(self._quarantine)

    def reap_pending_failures(self) -> int:
        """Drop the buffers of failed runs whose device work has finished; returns how many were released."""

        def ready(completion: object | None) -> bool:
            query = getattr(completion, "query", None)
            return True if not callable(query) else bool(query())

        with self._lock:
            kept = [item for item in self._quarantine if not ready(item[1])]
            released = len(self._quarantine) - len(kept)
            self._quarantine = kept
            return released

    def run(self, tensor: object) -> CompletionWork:
        self.reap_pending_failures()
        value, dependency = tensor, None
        resources: list[object] = [tensor]
        for stage in self.stages:
            try:
                execution = stage.launch(value, dependency)
            except BaseException:
                # kernels of earlier stages may still be reading these buffers: keep them until an event says so
                with self._lock:
                    self._quarantine.append(((*resources, value), stage.emergency_completion()))
                raise
            value, dependency = execution.value, execution.completion
            resources.extend(execution.resources)
        return CompletionWork(value, completion=dependency, resources=tuple(resources))


# ---- topology ----------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RankTopology:
    local_ranks: tuple[int, ...]
    inter_ranks: tuple[int, ...]


def rank_topology(context: CompileContext) -> RankTopology:
    """Ranks of my node and ranks that share my local index, from the context's topology fields."""

    if context.local_rank is None or context.local_world_size is None:
        raise ValueError("hierarchical compilation requires local rank and world size")
    if context.node_id is None or context.node_count is None:
        raise ValueError("hierarchical compilation requires node id and node count")
    L, nodes = context.local_world_size, context.node_count
    if context.world_size != L * nodes:
        raise ValueError("world size must equal local world size multiplied by node count")
    first = context.node_id * L
    if not first <= context.rank < first + L or context.local_rank != context.rank - first:
        raise ValueError("global rank is inconsistent with node and local rank metadata")
    return RankTopology(tuple(range(first, first + L)), tuple(n * L + context.local_rank for n in range(nodes)))


def all_hierarchy_groups(context: CompileContext) -> tuple[tuple[int, ...], ...]:
    """Every local group, then every inter group: the order in which all ranks must create them."""

    if context.local_world_size is None or context.node_count is None:
        raise ValueError("hierarchical group creation requires complete topology metadata")
    L, nodes = context.local_world_size, context.node_count
    local = tuple(tuple(range(n * L, (n + 1) * L)) for n in range(nodes))
    inter = tuple(tuple(n * L + i for n in range(nodes)) for i in range(L))
    return (*local, *inter)


def canonical_hierarchical_stages(compression: Any, *, inter_strategy: str = "topology",
                                  gather_strategy: str = "native_nccl") -> tuple[CommunicationStage, ...]:
    """The three stages of the chain, ready to put into `CommunicationPlan(strategy="hierarchical", stages=...)`."""

    return (
        CommunicationStage("local_reduce_scatter", "reduce_scatter", "compressed", compression=compression,
                           output_layout="shard", async_op=False),
        CommunicationStage("inter_all_reduce", "all_reduce", inter_strategy, compression=compression,
                           output_layout="shard", async_op=False),
        CommunicationStage("local_all_gather", "all_gather", gather_strategy,
                           compression=compression if gather_strategy != "native_nccl" else None,
                           output_layout="full", async_op=False),
    )


def _check_chain(plan: CommunicationPlan) -> None:
    problem = None
    if plan.collective != "all_reduce" or plan.output_layout != "full" or len(plan.stages) != 3:
        problem = "an all_reduce with full output and three stages is required"
    else:
        first, second, third = plan.stages
        if (first.collective, first.strategy, first.output_layout) != ("reduce_scatter", "compressed", "shard"):
            problem = "stage 1 must be a compressed reduce_scatter producing a shard"
        elif second.collective != "all_reduce" or second.output_layout != "shard" \
                or second.strategy not in _INTER_STRATEGIES:
            problem = "stage 2 must be an all_reduce of the shard"
        elif third.collective != "all_gather" or third.output_layout != "full" \
                or third.strategy not in _GATHER_STRATEGIES:
            problem = "stage 3 must be an all_gather restoring the full tensor"
        elif any(stage.async_op for stage in plan.stages):
            problem = "stages run inside one asynchronous chain and must not be asynchronous themselves"
    if problem is not None:
        raise ValueError("hierarchical execution requires the three-stage chain compressed reduce_scatter "
                         f"full->shard, all_reduce shard->shard, all_gather shard->full: {problem}")


def _numel(shape: tuple[int, ...]) -> int:
    total = 1
    for d in shape:
        total *= d
    return total


def compile_hierarchical_stages(plan: CommunicationPlan, context: CompileContext, *,
                                operation_factory: Callable[[CommunicationStage, CompileContext], Callable[..., Any]],
                                group_members: Callable[[object], Sequence[int]] | None = None,
                                group_factory: Callable[[tuple[int, ...]], object] | None = None,
                                stream_factory: Callable[[CommunicationStage, CompileContext], object] | None = None,
                                completion_factory: Callable[[object | None], object] | None = None,
                                ) -> HierarchicalExecutor:
    """Bind the three stages for the rank described by `context`.

    `operation_factory(stage, stage_context)` receives a context whose rank, world size, shape and process
    group are those of the stage's own group.  `group_members(group)` lists a group's global ranks
    (default: torch.distributed.get_process_group_ranks).  With `group_factory`, groups that the plan and
    the context do not supply are created: all of them, in the same order on every rank, because group
    creation is collective.
    """

    if plan.strategy != "hierarchical":
        raise ValueError("hierarchical stage compilation requires strategy='hierarchical'")
    if not callable(operation_factory):
        raise TypeError("operation_factory must be callable")
    _check_chain(plan)
    topology = rank_topology(context)
    members = group_members or _torch_group_members
    created: dict[tuple[int, ...], object] = {}
    missing = any(s.process_group is None and s.name not in context.process_groups for s in plan.stages)
    if group_factory is not None and missing:
        for ranks in all_hierarchy_groups(context):
            created.setdefault(ranks, group_factory(ranks))
    layout, shape = "full", tuple(context.shape)
    compiled = []
    for stage in plan.stages:
        scope = _TRANSITIONS.get((stage.collective, layout, stage.output_layout))
        if scope is None:
            raise UnsupportedCollective(f"hierarchical:{stage.name}",
                                        reason=f"unsupported stage transition {stage.collective}:{layout}->"
                                               f"{stage.output_layout}")
        expected = topology.local_ranks if scope == "local" else topology.inter_ranks
        group = stage.process_group if stage.process_group is not None else context.process_groups.get(stage.name)
        if group is None:
            if group_factory is None:
                raise ValueError(f"stage {stage.name!r} requires a compile-time process group or group factory")
            if expected not in created:
                created[expected] = group_factory(expected)
            group = created[expected]
        actual = tuple(int(r) for r in members(group))
        if actual != expected:
            raise ValueError(f"stage {stage.name!r} process group members {actual} do not match expected ranks "
                             f"{expected}")
        stage_context = replace(context, rank=expected.index(context.rank), world_size=len(expected), shape=shape,
                                process_group=group, process_groups={}, local_rank=None, local_world_size=None,
                                node_id=None, node_count=None)
        compiled.append(CompiledStage(
            name=stage.name, input_layout=layout, output_layout=stage.output_layout, participants=expected,
            process_group=group, operation=operation_factory(stage, stage_context),
            stream=None if stream_factory is None else stream_factory(stage, stage_context),
            completion_factory=completion_factory))
        if stage.collective == "reduce_scatter":
            shape = (-(-_numel(shape) // len(expected)),)
        elif stage.collective == "all_gather":
            shape = tuple(context.shape)
        layout = stage.output_layout
    if layout != plan.output_layout:
        raise ValueError(f"hierarchical final output layout {layout!r} does not match plan output layout "
                         f"{plan.output_layout!r}")
    return HierarchicalExecutor(compiled)


def _torch_group_members(group: object) -> tuple[int, ...]:
    from importlib import import_module

    dist = import_module("torch.distributed")
    getter = getattr(dist, "get_process_group_ranks", None)
    if not callable(getter):
        raise RuntimeError("torch.distributed.get_process_group_ranks is required for hierarchical compilation")
    return tuple(int(r) for r in getter(group))
