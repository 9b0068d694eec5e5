"""Torch-free control plane (plans, registry, compiler, work objects)."""

from .backend import AutoStrategySelector, BackendCapabilities, CommunicationBackend, StrategyChoice
from .chunking import ChunkPlan, ChunkRange, GroupShardPlan, compile_chunk_plan, hierarchy_groups
from .compiler import CompileCache, ResolvedPlan, compile, default_registry, resolve_plan
from .executor import CompileCacheKey, CompiledCommunicationPlan, CompiledExecutor, ObjectIdentity
from .hierarchy import (CompiledStage, HierarchicalExecutor, StageExecution, canonical_hierarchical_stages,
                        compile_hierarchical_stages)
from .info import ExecutionCounters, ExecutionCounterSnapshot, ExecutionInfo
from .plan import CommunicationPlan, CommunicationStage, CompileContext, WorkspacePolicy
from .registry import BackendKey, BackendRegistry
from .schedules import (ButterflySchedule, DirectExchangeSchedule, GatherTile, PairwiseSchedule, PairwiseStep,
                        PipelinedRingSchedule, RingAllGatherStep, RingReduceScatterStep, TreeEdge, TreeSchedule,
                        compile_butterfly_schedule, compile_direct_exchange_schedule, compile_pairwise_schedule,
                        compile_pipelined_ring_schedule, compile_tree_schedule, gather_tiles)
from .shard import ReducedShard
from .work import (BoundCollectiveWork, CollectiveWork, CompletionWork, ImmediateWork,
                   bind_execution_work)

__all__ = [name for name in dir() if not name.startswith("_")]
