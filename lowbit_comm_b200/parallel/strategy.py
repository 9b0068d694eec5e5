"""DDP-level strategy planner (torch-free).

Parity: ccdl_comm/communication/strategy.py:11-177 — same inputs, outputs and
decisions (world <= 2 -> all_gather; multi-node -> hierarchical when the
transport and process groups exist; single node -> reduce_scatter when
available; otherwise fall back to all_gather with a reason).  Added: the
`native_nccl` strategy name (uncompressed pass-through).
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..exceptions import UnsupportedCollective

SUPPORTED_STRATEGIES = frozenset({"auto", "all_gather", "all_reduce", "reduce_scatter", "hierarchical", "topology",
                                  "native_nccl"})
_NEEDS_CAPABILITY = ("hierarchical", "reduce_scatter", "topology")


@dataclass(frozen=True)
class TopologyInfo:
    rank: int
    world_size: int
    local_rank: int | None = None
    local_world_size: int | None = None
    node_id: int | None = None
    node_count: int | None = None
    intra_node: str = "unknown"
    inter_node: str = "unknown"
    has_process_groups: bool = False


@dataclass(frozen=True)
class CollectiveCapabilities:
    reduce_scatter: bool = False
    hierarchical: bool = False
    topology: bool = False
    hierarchical_recommended: bool = False
    fused_dequant_reduce: bool = False
    capability_flags: dict[str, bool] = field(default_factory=dict)

    def flags(self) -> dict[str, bool]:
        out = {name: getattr(self, name) for name in
               ("reduce_scatter", "hierarchical", "topology", "hierarchical_recommended", "fused_dequant_reduce")}
        out.update(self.capability_flags)
        return out


@dataclass(frozen=True)
class StrategyPlan:
    requested_strategy: str
    strategy: str
    fallback_strategy: str
    reason: str
    requires_fallback: bool
    capability_flags: dict[str, bool]


def plan_ddp_compression_strategy(*, requested_strategy: str, world_size: int, rank: int = 0,
                                  local_world_size: int | None = None, node_count: int | None = None,
                                  bucket_numel: int = 0, topology: TopologyInfo | None = None,
                                  capabilities: CollectiveCapabilities | None = None) -> StrategyPlan:
    del bucket_numel  # accepted for signature parity; sizes are handled by the strategy table
    wanted = requested_strategy.strip().lower()
    if wanted not in SUPPORTED_STRATEGIES:
        raise UnsupportedCollective(requested_strategy,
                                    reason="explicit strategy is unknown and no fallback was declared")
    caps = capabilities or CollectiveCapabilities()
    flags = caps.flags()
    if wanted in _NEEDS_CAPABILITY and not getattr(caps, wanted):
        raise UnsupportedCollective(wanted, reason=f"{wanted} transport unavailable for explicit strategy")

    def chosen(strategy: str, why: str, fallback: bool = False) -> StrategyPlan:
        return StrategyPlan(wanted, strategy, "all_gather", why, fallback, flags)

    if wanted != "auto":
        return chosen(wanted, f"explicit strategy {wanted}")
    topo = topology or TopologyInfo(rank=rank, world_size=world_size, local_world_size=local_world_size,
                                    node_count=node_count)
    nodes = topo.node_count if topo.node_count is not None else node_count
    if world_size <= 2:
        return chosen("all_gather", "world_size<=2 uses validated all_gather path")
    if nodes is not None and nodes > 1:
        if not caps.hierarchical:
            return chosen("all_gather", "multi-node hierarchical unavailable; falling back to all_gather", True)
        if not topo.has_process_groups:
            return chosen("all_gather", "process groups unavailable for multi-node hierarchical strategy; "
                                        "falling back to all_gather", True)
        return chosen("hierarchical", "multi-node hierarchical strategy selected")
    if caps.reduce_scatter:
        return chosen("reduce_scatter", "single-node capable reduce_scatter strategy selected")
    if caps.hierarchical and caps.hierarchical_recommended:
        return chosen("hierarchical", "single-node hierarchical strategy selected")
    if caps.hierarchical:
        return chosen("all_gather", "hierarchical transport is not performance-recommended for single-node auto "
                                    "strategy; falling back to all_gather", True)
    return chosen("all_gather", "reduce_scatter and hierarchical unavailable for single-node auto strategy; "
                                "falling back to all_gather", True)
