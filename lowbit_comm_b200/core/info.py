"""What a compiled plan will do (decided before any launch) and what it has done so far (counters).

`ExecutionInfo` is immutable and attached to every compiled plan, executor and work object; `ExecutionCounters`
is shared by an executor and the work objects it hands out.  Field names follow the reference
(ccdl_comm/execution_info.py:13-110).
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass, field, replace
from typing import NamedTuple

from ._checks import freeze, need_texts, read_only, text_tuple


@dataclass(frozen=True)
class ExecutionInfo:
    requested_strategy: str
    executed_strategy: str
    backend: str
    fallback_used: bool
    fallback_reason: str | None
    stage_names: tuple[str, ...]
    original_bytes: int
    compressed_bytes: int
    compression_ratio: float
    workspace_cache_hit: bool
    async_capable: bool
    fast_path: str
    details: Mapping[str, object] = field(default_factory=dict)

    def __post_init__(self) -> None:
        need_texts(self, "requested_strategy", "executed_strategy", "backend", "fast_path")
        for name in ("original_bytes", "compressed_bytes"):
            if getattr(self, name) < 0:
                raise ValueError(f"{name} must be >= 0")
        if not (math.isfinite(self.compression_ratio) and self.compression_ratio > 0.0):
            raise ValueError("compression_ratio must be finite and > 0")
        # a fallback always says why; no fallback never carries a reason
        explained = bool(self.fallback_reason and self.fallback_reason.strip())
        if self.fallback_used and not explained:
            raise ValueError("fallback_reason is required when fallback_used is true")
        if not self.fallback_used and self.fallback_reason is not None:
            raise ValueError("fallback_reason must be None when fallback_used is false")
        freeze(self, details=read_only(self.details),
               stage_names=text_tuple(self.stage_names, "stage_names", message="stage name must be a non-empty string"))

    @property
    def saved_bytes(self) -> int:
        """Bytes that do not cross the wire because of compression (never negative)."""

        return max(0, self.original_bytes - self.compressed_bytes)

    def with_details(self, **more: object) -> "ExecutionInfo":
        """A copy whose `details` also hold `more` (existing keys are overwritten)."""

        return replace(self, details={**dict(self.details), **more})

    def summary(self) -> str:
        """One line for logs: strategy (and fallback), backend, path, bytes."""

        route = self.executed_strategy if not self.fallback_used else \
            f"{self.requested_strategy} -> {self.executed_strategy} ({self.fallback_reason})"
        stages = f" [{' > '.join(self.stage_names)}]" if len(self.stage_names) > 1 else ""
        return (f"{route} on {self.backend} via {self.fast_path}{stages}: {self.original_bytes} -> "
                f"{self.compressed_bytes} bytes ({self.compression_ratio:.2f}x)")


class ExecutionCounterSnapshot(NamedTuple):
    run_calls: int
    completed_runs: int
    failed_runs: int
    wait_calls: int
    query_calls: int

    @property
    def in_flight(self) -> int:
        """Runs that have neither completed nor failed yet."""

        return self.run_calls - self.completed_runs - self.failed_runs


class ExecutionCounters:
    """Five integers shared by an executor and the work it returns.  Diagnostics only: increments are plain
    `+=` and not synchronised across threads."""

    __slots__ = ("_n",)
    _SLOTS = {"run": 0, "completed": 1, "failed": 2, "wait": 3, "query": 4}

    def __init__(self) -> None:
        self._n = [0] * len(self._SLOTS)

    def snapshot(self) -> ExecutionCounterSnapshot:
        return ExecutionCounterSnapshot(*self._n)

    def _bump(self, what: str) -> None:
        self._n[self._SLOTS[what]] += 1

    def _record_run(self) -> None:
        self._bump("run")

    def _record_completed(self) -> None:
        self._bump("completed")

    def _record_failed(self) -> None:
        self._bump("failed")

    def _record_wait(self) -> None:
        self._bump("wait")

    def _record_query(self) -> None:
        self._bump("query")
