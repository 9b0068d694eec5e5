"""Planner that groups adjacent gradient buckets for one fused launch.

Parity: ccdl_comm/communication/bucket_fusion.py:11-177 (same inputs, outputs
and rules: consecutive buckets only, bounded element count and bucket count,
same dtype unless told otherwise, "full bucket" consumers stay alone).  It is a
scheduling contract; a transport may use or ignore the plan.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

DEFAULT_MAX_FUSED_BUCKET_NUMEL = 4_000_000
DEFAULT_MAX_FUSED_BUCKET_COUNT = 8


@dataclass(frozen=True)
class BucketDescriptor:
    index: int
    numel: int
    dtype: str = "auto"
    shape: tuple[int, ...] = ()
    requires_full_bucket: bool = False
    metadata: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class BucketFusionGroup:
    bucket_indices: tuple[int, ...]
    total_numel: int
    dtype: str
    fused: bool
    reason: str

    def to_metadata(self) -> dict[str, Any]:
        return dict(bucket_indices=self.bucket_indices, total_numel=self.total_numel, dtype=self.dtype,
                    fused=self.fused, reason=self.reason)


@dataclass(frozen=True)
class BucketFusionPlan:
    enabled: bool
    groups: tuple[BucketFusionGroup, ...]

    def _count(self, fused: bool, what=len) -> int:
        return sum(what(g.bucket_indices) for g in self.groups if g.fused is fused)

    @property
    def group_count(self) -> int:
        return len(self.groups)

    @property
    def fused_group_count(self) -> int:
        return sum(1 for g in self.groups if g.fused)

    @property
    def fused_bucket_count(self) -> int:
        return self._count(True)

    @property
    def skipped_bucket_count(self) -> int:
        return self._count(False)

    @property
    def total_fused_numel(self) -> int:
        return sum(g.total_numel for g in self.groups if g.fused)

    def to_metadata(self) -> dict[str, Any]:
        return {"enabled": self.enabled, "group_count": self.group_count,
                "fused_group_count": self.fused_group_count, "fused_bucket_count": self.fused_bucket_count,
                "skipped_bucket_count": self.skipped_bucket_count, "total_fused_numel": self.total_fused_numel,
                "groups": [g.to_metadata() for g in self.groups]}


def _alone(bucket: BucketDescriptor, why: str) -> BucketFusionGroup:
    return BucketFusionGroup((bucket.index,), bucket.numel, bucket.dtype, False, why)


def _close(run: list[BucketDescriptor]) -> BucketFusionGroup:
    many = len(run) > 1
    return BucketFusionGroup(tuple(b.index for b in run), sum(b.numel for b in run), run[0].dtype, many,
                             "compatible adjacent buckets" if many else "single compatible bucket")


def plan_bucket_fusion(buckets: Sequence[BucketDescriptor], *, enabled: bool = True,
                       max_fused_numel: int = DEFAULT_MAX_FUSED_BUCKET_NUMEL,
                       max_bucket_count: int = DEFAULT_MAX_FUSED_BUCKET_COUNT,
                       require_same_dtype: bool = True) -> BucketFusionPlan:
    if max_fused_numel <= 0:
        raise ValueError("max_fused_numel must be positive")
    if max_bucket_count <= 0:
        raise ValueError("max_bucket_count must be positive")
    out: list[BucketFusionGroup] = []
    run: list[BucketDescriptor] = []
    for b in buckets:
        if b.numel <= 0:
            raise ValueError("bucket numel must be positive")
        if not enabled:
            out.append(_alone(b, "fusion disabled"))
            continue
        if b.requires_full_bucket:
            if run:
                out.append(_close(run))
                run = []
            out.append(_alone(b, "requires full-bucket consumer"))
            continue
        fits = bool(run) and len(run) < max_bucket_count \
            and sum(x.numel for x in run) + b.numel <= max_fused_numel \
            and (not require_same_dtype or b.dtype == run[-1].dtype)
        if run and not fits:
            out.append(_close(run))
            run = []
        run.append(b)
    if run:
        out.append(_close(run))
    return BucketFusionPlan(enabled, tuple(out))
