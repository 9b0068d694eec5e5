"""Planner that groups adjacent gradient buckets for one fused launch.

Parity: ccdl_comm/communication/bucket_fusion.py:11-177 (same inputs, outputs
and rules: consecutive buckets only, bounded element count and bucket count,
same dtype unless told otherwise, "full bucket" consumers stay alone).  It is a
scheduling contract; a transport may use or ignore the plan.

The planner is one pass over the buckets with a `_Run` that accumulates the open group; `launches_saved`
(an addition) is what a fused transport gains: one collective per group instead of one per bucket, which on
NVSwitch is a latency saving, not a bandwidth one.
"""

from __future__ import annotations

from collections.abc import Iterable, Iterator
from dataclasses import asdict, dataclass, field
from typing import Any

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
        return asdict(self)


_TALLY_NAMES = ("group_count", "fused_group_count", "fused_bucket_count", "skipped_bucket_count", "total_fused_numel")


@dataclass(frozen=True)
class BucketFusionPlan:
    enabled: bool
    groups: tuple[BucketFusionGroup, ...]

    def _tally(self) -> dict[str, int]:
        tally = dict.fromkeys(_TALLY_NAMES, 0)
        for group in self.groups:
            members = len(group.bucket_indices)
            tally["group_count"] += 1
            if group.fused:
                tally["fused_group_count"] += 1
                tally["fused_bucket_count"] += members
                tally["total_fused_numel"] += group.total_numel
            else:
                tally["skipped_bucket_count"] += members
        return tally

    group_count = property(lambda self: len(self.groups))
    fused_group_count = property(lambda self: self._tally()["fused_group_count"])
    fused_bucket_count = property(lambda self: self._tally()["fused_bucket_count"])
    skipped_bucket_count = property(lambda self: self._tally()["skipped_bucket_count"])
    total_fused_numel = property(lambda self: self._tally()["total_fused_numel"])

    @property
    def launches_saved(self) -> int:
        """Collectives a transport that honours the plan does not have to launch."""

        tally = self._tally()
        return tally["fused_bucket_count"] - tally["fused_group_count"]

    def to_metadata(self) -> dict[str, Any]:
        return {"enabled": self.enabled, **self._tally(), "groups": [g.to_metadata() for g in self.groups]}


class _Run:
    """The group that is still open: consecutive buckets that may share one launch."""

    def __init__(self, numel_limit: int, count_limit: int, same_dtype: bool) -> None:
        self._limits = (numel_limit, count_limit, same_dtype)
        self._members: list[BucketDescriptor] = []
        self._numel = 0

    def admits(self, bucket: BucketDescriptor) -> bool:
        numel_limit, count_limit, same_dtype = self._limits
        if not self._members:
            return True
        return (len(self._members) < count_limit and self._numel + bucket.numel <= numel_limit
                and not (same_dtype and bucket.dtype != self._members[-1].dtype))

    def add(self, bucket: BucketDescriptor) -> None:
        self._members.append(bucket)
        self._numel += bucket.numel

    def close(self) -> Iterator[BucketFusionGroup]:
        """Yields the finished group (nothing when the run is empty) and starts a new run."""

        if self._members:
            several = len(self._members) > 1
            yield BucketFusionGroup(tuple(b.index for b in self._members), self._numel, self._members[0].dtype,
                                    several, "compatible adjacent buckets" if several else "single compatible bucket")
        self._members, self._numel = [], 0


def _alone(bucket: BucketDescriptor, why: str) -> BucketFusionGroup:
    return BucketFusionGroup((bucket.index,), bucket.numel, bucket.dtype, False, why)


def _groups(buckets: Iterable[BucketDescriptor], enabled: bool, run: _Run) -> Iterator[BucketFusionGroup]:
    for bucket in buckets:
        if bucket.numel <= 0:
            raise ValueError("bucket numel must be positive")
        if not enabled:
            yield _alone(bucket, "fusion disabled")
        elif bucket.requires_full_bucket:
            yield from run.close()
            yield _alone(bucket, "requires full-bucket consumer")
        else:
            if not run.admits(bucket):
                yield from run.close()
            run.add(bucket)
    yield from run.close()


def plan_bucket_fusion(buckets: Iterable[BucketDescriptor], *, enabled: bool = True,
                       max_fused_numel: int = DEFAULT_MAX_FUSED_BUCKET_NUMEL,
                       max_bucket_count: int = DEFAULT_MAX_FUSED_BUCKET_COUNT,
                       require_same_dtype: bool = True) -> BucketFusionPlan:
    for name, limit in (("max_fused_numel", max_fused_numel), ("max_bucket_count", max_bucket_count)):
        if limit <= 0:
            raise ValueError(f"{name} must be positive")
    run = _Run(max_fused_numel, max_bucket_count, require_same_dtype)
    return BucketFusionPlan(enabled, tuple(_groups(buckets, enabled, run)))
