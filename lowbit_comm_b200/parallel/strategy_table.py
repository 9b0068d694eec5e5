"""Benchmark-backed automatic strategy choice for B200.

Role parity: ccdl_comm/cuda/strategy_table.py:21-255 (immutable rules with
evidence, overlap rejection, explainable `StrategyChoice`, adapter to the
registry's selector protocol).  The reference's only rule set is RTX A6000 /
fp16 / W in {2,4}; this table carries rules measured on B200 with the sweep in
`benchmarks/allreduce_sweep.py` (summaries under `profiles/`).

Rule of thumb the measurements support on NVLink 5: the one-stage path (every
rank reduces W payloads) wins for W <= 2 and for small tensors, where launch
count dominates; the two-stage path wins for W >= 4 above a few MiB because it
moves 2(W-1)/W payloads instead of W-1.  Full-output rules start at the size
from which the fused path was measured faster than NCCL's bf16 all-reduce
(`B200_CROSSOVER_NUMEL`); below it, and below `min_compress_numel` elements in
any case, `auto` keeps the uncompressed NCCL all-reduce, which is exact.
"""

from __future__ import annotations

import math
from collections.abc import Callable
from dataclasses import dataclass
from typing import NamedTuple

from ..config import CompressionConfig
from ..core.backend import StrategyChoice
from ..core.compiler import normalize_dtype
from ..core.plan import CommunicationPlan, CompileContext
from ..exceptions import UnsupportedCollective

B200_POLICY_ID = "b200-nvlink5-v1"
B200_EVIDENCE = "profiles/allreduce_sweep_b200.md"
PRODUCTION_PROFILE = CompressionConfig(bit=8, group_size=64)


def _numel(shape: tuple[int, ...]) -> int:
    return math.prod(shape)


def normalize_architecture(value: str) -> str:
    return "_".join(value.strip().lower().replace("-", " ").split())


def _profile(compression: CompressionConfig) -> tuple:
    """The part of a compression config that changes the wire format (error-feedback settings do not)."""

    return (compression.bit, compression.group_size, compression.topk, compression.quant_type)


class RuleDomain(NamedTuple):
    """Everything a rule is measured for except the size range.  Rules of one domain must not overlap."""

    collective: str
    output_layout: str
    device_architecture: str
    world_size: int
    dtype: str
    profile: tuple

    @classmethod
    def of_request(cls, plan: CommunicationPlan, context: CompileContext) -> "RuleDomain":
        return cls(plan.collective, plan.output_layout, normalize_architecture(context.device_architecture),
                   context.world_size, normalize_dtype(context.dtype), _profile(plan.compression))


@dataclass(frozen=True)
class CudaStrategyRule:
    collective: str
    output_layout: str
    device_architecture: str
    world_size: int
    dtype: str
    compression: CompressionConfig
    min_numel: int
    max_numel: int
    strategy: str
    speedup: float
    same_semantics_baseline: bool

    def __post_init__(self) -> None:
        if self.min_numel < 0 or self.max_numel < self.min_numel:
            raise ValueError("strategy rule requires 0 <= min_numel <= max_numel")
        if self.speedup <= 0:
            raise ValueError("strategy rule speedup must be > 0")

    @property
    def domain(self) -> RuleDomain:
        return RuleDomain(self.collective, self.output_layout, self.device_architecture, self.world_size, self.dtype,
                          _profile(self.compression))

    def covers(self, numel: int) -> bool:
        return self.min_numel <= numel <= self.max_numel

    def overlaps(self, other: "CudaStrategyRule") -> bool:
        return self.domain == other.domain and (self.covers(other.min_numel) or other.covers(self.min_numel))

    def matches(self, context: CompileContext, compression: CompressionConfig, *, collective: str,
                output_layout: str) -> bool:
        asked = RuleDomain(collective, output_layout, normalize_architecture(context.device_architecture),
                           context.world_size, normalize_dtype(context.dtype), _profile(compression))
        return asked == self.domain and self.covers(_numel(context.shape))


_SERVED = {("all_reduce", "full"), ("reduce_scatter", "shard")}


class CudaStrategyTable:
    def __init__(self, rules: tuple[CudaStrategyRule, ...], *, policy_id: str = B200_POLICY_ID,
                 evidence: str = B200_EVIDENCE, min_compress_numel: int = 262_144) -> None:
        self._rules = tuple(rules)
        self.policy_id, self.evidence, self.min_compress_numel = policy_id, evidence, min_compress_numel
        self._by_domain: dict[RuleDomain, list[CudaStrategyRule]] = {}
        for rule in self._rules:
            same_domain = self._by_domain.setdefault(rule.domain, [])
            if any(rule.overlaps(earlier) for earlier in same_domain):
                raise ValueError("CUDA strategy table contains overlapping rules")
            same_domain.append(rule)

    @property
    def rules(self) -> tuple[CudaStrategyRule, ...]:
        return self._rules

    # Elements (16-bit) from which the fused all-reduce was measured faster than NCCL's bf16 all-reduce on B200:
    # 2 MiB on 2 GPUs, 128 MiB on 4, 64 MiB on 8 (profiles/allreduce_sweep_b200.md).  Below it `auto` keeps NCCL.
    B200_CROSSOVER_NUMEL = {2: 1 << 20, 4: 1 << 26, 8: 1 << 25}

    @classmethod
    def for_b200(cls, measured: dict | None = None) -> "CudaStrategyTable":
        """Rules for sm_100 / bf16+fp16 / W in {2,4,8}; `measured` overrides the recorded speed-ups
        (keys `(layout, world)` -> speed-up over the NCCL bf16 full all-reduce)."""

        # Recorded on this pool's B200s (bf16, int8 group 64, error feedback on; profiles/allreduce_sweep_b200.md).
        # full: NCCL bf16 all-reduce time / best fused path at 256 MiB.  shard: NCCL *full* all-reduce time /
        # (K1 + K2) of the two-stage path at 64 MiB, the baseline the reference's own table uses for shards.
        recorded = {("full", 2): 1.20, ("full", 4): 1.25, ("full", 8): 1.17,
                    ("shard", 2): 1.5, ("shard", 4): 1.5, ("shard", 8): 1.7}
        recorded.update(measured or {})
        rules = []
        for (layout, world), speedup in recorded.items():
            for dtype in ("bf16", "fp16"):
                common = dict(collective="all_reduce" if layout == "full" else "reduce_scatter", output_layout=layout,
                              device_architecture="sm_100", world_size=world, dtype=dtype,
                              compression=PRODUCTION_PROFILE, speedup=speedup,
                              same_semantics_baseline=layout == "full")
                if layout == "shard":
                    rules.append(CudaStrategyRule(min_numel=262_144, max_numel=1 << 31, strategy="compressed", **common))
                    continue
                # full output: compressed only from the size at which it was measured to beat NCCL's bf16 all-reduce
                start = cls.B200_CROSSOVER_NUMEL.get(world, 1 << 25)
                # one stage while tensor bytes x W <= 64 MiB (measured: 16 MiB on 4 GPUs, 8 MiB on 8), and always for W <= 2
                one_stage_max = (1 << 31) if world <= 2 else (64 << 20) // (2 * world)
                if start <= one_stage_max:
                    rules.append(CudaStrategyRule(min_numel=start, max_numel=one_stage_max, strategy="all_gather", **common))
                if one_stage_max < 1 << 31:
                    rules.append(CudaStrategyRule(min_numel=max(start, one_stage_max + 1), max_numel=1 << 31,
                                                  strategy="reduce_scatter", **common))
        return cls(tuple(rules))

    @classmethod
    def from_task13_a6000(cls) -> "CudaStrategyTable":
        """The reference's own table, for callers that ask for it by name: RTX A6000, fp16, 2 and 4 GPUs,
        8 Mi - 32 Mi elements, `topology` for full output and `compressed` for shard output, with the
        speed-ups its Task 13 report published (ccdl_comm/cuda/strategy_table.py:81-107).  Nothing on a B200
        matches these rules; `for_b200` is the table the CUDA backend registers."""

        published = {("full", 2): 1.6253136683796892, ("full", 4): 1.33102168223003,
                     ("shard", 2): 2.855439327752976, ("shard", 4): 2.6032121073325847}
        rules = tuple(
            CudaStrategyRule(collective="all_reduce" if layout == "full" else "reduce_scatter", output_layout=layout,
                             device_architecture="nvidia_rtx_a6000", world_size=world, dtype="fp16",
                             compression=PRODUCTION_PROFILE, min_numel=8_388_608, max_numel=33_554_432,
                             strategy="topology" if layout == "full" else "compressed", speedup=speedup,
                             same_semantics_baseline=layout == "full")
            for (layout, world), speedup in published.items())
        return cls(rules, policy_id="cuda-task13-a6000-v1", evidence="tests/benchmarks/reports/task13_topology")

    # -- selection --------------------------------------------------------------------------------------
    def lookup(self, plan: CommunicationPlan, context: CompileContext) -> CudaStrategyRule | None:
        """The measured rule that covers this request exactly, if there is one."""

        numel = _numel(context.shape)
        candidates = self._by_domain.get(RuleDomain.of_request(plan, context), ())
        return next((rule for rule in candidates if rule.covers(numel)), None)

    def select(self, plan: CommunicationPlan, context: CompileContext) -> StrategyChoice:
        if not isinstance(plan, CommunicationPlan):
            raise TypeError("plan must be a CommunicationPlan")
        if not isinstance(context, CompileContext):
            raise TypeError("context must be a CompileContext")
        if plan.compression is None:
            return self._unmeasured("native_nccl", "uncompressed auto request uses native NCCL")
        if (plan.collective, plan.output_layout) not in _SERVED:
            raise UnsupportedCollective(f"{plan.collective}:{plan.output_layout}",
                                        reason="CUDA strategy table has no safe semantics for this request")
        rule = self.lookup(plan, context)
        if rule is not None:
            return self._measured(rule)
        if plan.output_layout == "shard":
            return self._unmeasured("compressed", "unverified sharded dimensions retain the only registered "
                                                  "semantically compatible ReducedShard transport")
        if _numel(context.shape) < self.min_compress_numel:
            return self._unmeasured("native_nccl", "small bucket uses uncompressed NCCL: launch latency dominates "
                                                   f"below {self.min_compress_numel} elements")
        if not self._mismatches(context, plan.compression, quiet=True):
            return self._unmeasured("native_nccl", "below the measured crossover uncompressed NCCL is as fast or "
                                                   "faster: the size is outside every rule of this world size")
        return self._unmeasured("native_nccl", "unverified dimensions use safe uncompressed NCCL: "
                                + ", ".join(self._mismatches(context, plan.compression)))

    def _unmeasured(self, strategy: str, why: str) -> StrategyChoice:
        return StrategyChoice(strategy, why, self.policy_id, False)

    def _measured(self, rule: CudaStrategyRule) -> StrategyChoice:
        """A full-output rule compares like with like (expected speed-up, NCCL as the way back); a shard rule
        is measured against NCCL's *full* all-reduce, so its speed-up is an observation with a named baseline."""

        why = (f"benchmark table {self.policy_id} matched all validated dimensions; "
               f"observed speedup {rule.speedup:.2f}x")
        if rule.same_semantics_baseline:
            kind = {"expected_speedup": rule.speedup}
        else:
            kind = {"observed_speedup": rule.speedup, "baseline": "nccl_bf16_full_output_reference"}
        return StrategyChoice(rule.strategy, why, self.policy_id, True, evidence=self.evidence,
                              fallback=("native_nccl",) if rule.output_layout == "full" else (), **kind)

    def _mismatches(self, context: CompileContext, comp: CompressionConfig, *, quiet: bool = False) -> tuple[str, ...]:
        """Which dimensions of the request no rule of this table was measured for (`quiet`: an empty tuple
        instead of the "unmatched_rule" placeholder when every dimension is known)."""

        measured = {name: {getattr(rule, name) for rule in self._rules}
                    for name in ("device_architecture", "world_size", "dtype")}
        asked = {"device_architecture": normalize_architecture(context.device_architecture),
                 "world_size": context.world_size, "dtype": normalize_dtype(context.dtype)}
        missing = [name for name, value in asked.items() if value not in measured[name]]
        if _profile(comp) not in {_profile(rule.compression) for rule in self._rules}:
            missing.append("compression_profile")
        return tuple(missing) or (() if quiet else ("unmatched_rule",))

    def as_selector(self) -> Callable[[CommunicationPlan, CompileContext], StrategyChoice]:
        return self.select
