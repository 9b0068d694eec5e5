"""Which collective a DDP gradient hook should use (torch-free).

The automatic choice is an ordered rule table (`_AUTO_RULES`): the first rule whose condition holds for the
job's shape and the transports that exist names the strategy and says why; a rule that settles for
`all_gather` because something better is missing marks the plan as a fallback.  Inputs, outputs, decisions
and reason texts are the reference's (ccdl_comm/communication/strategy.py:11-177).  Added: the `native_nccl`
strategy name (uncompressed pass-through).
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field
from typing import NamedTuple

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


class _Job(NamedTuple):
    """What the automatic rules look at."""

    world_size: int
    nodes: int | None
    has_process_groups: bool
    caps: CollectiveCapabilities

    @property
    def multi_node(self) -> bool:
        return self.nodes is not None and self.nodes > 1


class _Rule(NamedTuple):
    applies: Callable[[_Job], bool]
    strategy: str
    reason: str
    settles: bool = False        # True: all_gather chosen because the better transport is missing


_AUTO_RULES: tuple[_Rule, ...] = (
    _Rule(lambda j: j.world_size <= 2, "all_gather", "world_size<=2 uses validated all_gather path"),
    # more than one node
    _Rule(lambda j: j.multi_node and not j.caps.hierarchical, "all_gather",
          "multi-node hierarchical unavailable; falling back to all_gather", True),
    _Rule(lambda j: j.multi_node and not j.has_process_groups, "all_gather",
          "process groups unavailable for multi-node hierarchical strategy; falling back to all_gather", True),
    _Rule(lambda j: j.multi_node, "hierarchical", "multi-node hierarchical strategy selected"),
    # one node
    _Rule(lambda j: j.caps.reduce_scatter, "reduce_scatter", "single-node capable reduce_scatter strategy selected"),
    _Rule(lambda j: j.caps.hierarchical and j.caps.hierarchical_recommended, "hierarchical",
          "single-node hierarchical strategy selected"),
    _Rule(lambda j: j.caps.hierarchical, "all_gather",
          "hierarchical transport is not performance-recommended for single-node auto strategy; "
          "falling back to all_gather", True),
    _Rule(lambda j: True, "all_gather",
          "reduce_scatter and hierarchical unavailable for single-node auto strategy; falling back to all_gather",
          True),
)


def plan_ddp_compression_strategy(*, requested_strategy: str, world_size: int, rank: int = 0,
                                  local_world_size: int | None = None, node_count: int | None = None,
                                  bucket_numel: int = 0, topology: TopologyInfo | None = None,
                                  capabilities: CollectiveCapabilities | None = None) -> StrategyPlan:
    """`bucket_numel`, `rank` and `local_world_size` are accepted for callers written against the reference;
    size-dependent choices are the strategy table's job."""

    wanted = requested_strategy.strip().lower()
    if wanted not in SUPPORTED_STRATEGIES:
        raise UnsupportedCollective(requested_strategy,
                                    reason="explicit strategy is unknown and no fallback was declared")
    caps = capabilities or CollectiveCapabilities()
    if wanted in _NEEDS_CAPABILITY and not getattr(caps, wanted):
        raise UnsupportedCollective(wanted, reason=f"{wanted} transport unavailable for explicit strategy")
    if wanted == "auto":
        nodes = topology.node_count if topology is not None and topology.node_count is not None else node_count
        job = _Job(world_size, nodes, bool(topology and topology.has_process_groups), caps)
        rule = next(r for r in _AUTO_RULES if r.applies(job))
        strategy, reason, settles = rule.strategy, rule.reason, rule.settles
    else:
        strategy, reason, settles = wanted, f"explicit strategy {wanted}", False
    return StrategyPlan(requested_strategy=wanted, strategy=strategy, fallback_strategy="all_gather", reason=reason,
                        requires_fallback=settles, capability_flags=caps.flags())
