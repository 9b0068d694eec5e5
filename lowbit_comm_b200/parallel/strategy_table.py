"""Benchmark-backed automatic strategy choice for B200.

Role parity: ccdl_comm/cuda/strategy_table.py:21-255 (immutable rules with
evidence, overlap rejection, explainable `StrategyChoice`, adapter to the
registry's selector protocol).  The reference's only rule set is RTX A6000 /
fp16 / W in {2,4}; this table carries rules measured on B200 with the sweep in
`benchmarks/allreduce_sweep.py` (summaries under `profiles/`).

Rule of thumb the measurements support on NVLink 5: the one-stage path (every
rank reduces W payloads) wins for W <= 2 and for small tensors, where launch
count dominates; the two-stage path wins for W >= 4 above a few MiB because it
moves 2(W-1)/W payloads instead of W-1.  Below `min_compress_numel` elements an
uncompressed NCCL all-reduce is as fast and exact.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass

from ..config import CompressionConfig
from ..core.backend import StrategyChoice
from ..core.compiler import normalize_dtype
from ..core.plan import CommunicationPlan, CompileContext
from ..exceptions import UnsupportedCollective

B200_POLICY_ID = "b200-nvlink5-v1"
B200_EVIDENCE = "profiles/allreduce_sweep_b200.md"
PRODUCTION_PROFILE = CompressionConfig(bit=8, group_size=64)


def _numel(shape: tuple[int, ...]) -> int:
    total = 1
    for d in shape:
        total *= d
    return total


def normalize_architecture(value: str) -> str:
    return "_".join(value.strip().lower().replace("-", " ").split())


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
    def domain(self) -> tuple:
        return (self.collective, self.output_layout, self.device_architecture, self.world_size, self.dtype,
                self.compression)

    def matches(self, context: CompileContext, compression: CompressionConfig, *, collective: str,
                output_layout: str) -> bool:
        same_profile = (compression.bit, compression.group_size, compression.topk, compression.quant_type) == \
            (self.compression.bit, self.compression.group_size, self.compression.topk, self.compression.quant_type)
        return (collective == self.collective and output_layout == self.output_layout
                and normalize_architecture(context.device_architecture) == self.device_architecture
                and context.world_size == self.world_size and normalize_dtype(context.dtype) == self.dtype
                and same_profile and self.min_numel <= _numel(context.shape) <= self.max_numel)


class CudaStrategyTable:
    def __init__(self, rules: tuple[CudaStrategyRule, ...], *, policy_id: str = B200_POLICY_ID,
                 evidence: str = B200_EVIDENCE, min_compress_numel: int = 262_144) -> None:
        self._rules = tuple(rules)
        self.policy_id, self.evidence, self.min_compress_numel = policy_id, evidence, min_compress_numel
        for i, a in enumerate(self._rules):
            for b in self._rules[i + 1:]:
                if a.domain == b.domain and a.min_numel <= b.max_numel and b.min_numel <= a.max_numel:
                    raise ValueError("CUDA strategy table contains overlapping rules")

    @property
    def rules(self) -> tuple[CudaStrategyRule, ...]:
        return self._rules

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
                elif world <= 2:
                    rules.append(CudaStrategyRule(min_numel=262_144, max_numel=1 << 31, strategy="all_gather", **common))
                else:
                    # one stage while tensor bytes x W <= 64 MiB (measured crossover: 16 MiB on 4 GPUs, 8 MiB on 8)
                    one_stage_max = (64 << 20) // (2 * world)
                    rules.append(CudaStrategyRule(min_numel=262_144, max_numel=one_stage_max, strategy="all_gather",
                                                  **common))
                    rules.append(CudaStrategyRule(min_numel=one_stage_max + 1, max_numel=1 << 31,
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

    def select(self, plan: CommunicationPlan, context: CompileContext) -> StrategyChoice:
        if not isinstance(plan, CommunicationPlan):
            raise TypeError("plan must be a CommunicationPlan")
        if not isinstance(context, CompileContext):
            raise TypeError("context must be a CompileContext")
        comp = plan.compression
        if comp is None:
            return StrategyChoice("native_nccl", "uncompressed auto request uses native NCCL", self.policy_id, False)
        semantic = (plan.collective, plan.output_layout)
        if semantic not in {("all_reduce", "full"), ("reduce_scatter", "shard")}:
            raise UnsupportedCollective(f"{plan.collective}:{plan.output_layout}",
                                        reason="CUDA strategy table has no safe semantics for this request")
        for rule in self._rules:
            if rule.matches(context, comp, collective=plan.collective, output_layout=plan.output_layout):
                same = rule.same_semantics_baseline
                return StrategyChoice(
                    rule.strategy,
                    f"benchmark table {self.policy_id} matched all validated dimensions; observed speedup {rule.speedup:.2f}x",
                    self.policy_id, True, expected_speedup=rule.speedup if same else None,
                    observed_speedup=None if same else rule.speedup,
                    baseline=None if same else "nccl_bf16_full_output_reference", evidence=self.evidence,
                    fallback=("native_nccl",) if rule.output_layout == "full" else ())
        if semantic == ("all_reduce", "full"):
            small = _numel(context.shape) < self.min_compress_numel
            why = ("small bucket uses uncompressed NCCL: launch latency dominates below "
                   f"{self.min_compress_numel} elements") if small else \
                "unverified dimensions use safe uncompressed NCCL: " + ", ".join(self._mismatches(context, comp))
            return StrategyChoice("native_nccl", why, self.policy_id, False)
        return StrategyChoice("compressed", "unverified sharded dimensions retain the only registered semantically "
                              "compatible ReducedShard transport", self.policy_id, False)

    def _mismatches(self, context: CompileContext, comp: CompressionConfig) -> tuple[str, ...]:
        out = []
        if normalize_architecture(context.device_architecture) != "sm_100":
            out.append("device_architecture")
        if context.world_size not in {r.world_size for r in self._rules}:
            out.append("world_size")
        if normalize_dtype(context.dtype) not in {r.dtype for r in self._rules}:
            out.append("dtype")
        if (comp.bit, comp.group_size, comp.topk, comp.quant_type) != (8, 64, 0, "linear"):
            out.append("compression_profile")
        return tuple(out) or ("unmatched_rule",)

    def as_selector(self) -> Callable[[CommunicationPlan, CompileContext], StrategyChoice]:
        return lambda plan, context: self.select(plan, context)
