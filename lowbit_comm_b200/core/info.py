"""Static execution metadata and cheap counters.

Parity: ccdl_comm/execution_info.py:13-110.
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass, field
from types import MappingProxyType
from typing import NamedTuple

from ._checks import need_text


@dataclass(frozen=True)
class ExecutionInfo:
    """What a compiled plan will do, decided before any launch."""

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
        for attr in ("requested_strategy", "executed_strategy", "backend", "fast_path"):
            need_text(getattr(self, attr), attr)
        names = tuple(self.stage_names)
        for name in names:
            need_text(name, "stage name")
        object.__setattr__(self, "stage_names", names)
        if self.original_bytes < 0:
            raise ValueError("original_bytes must be >= 0")
        if self.compressed_bytes < 0:
            raise ValueError("compressed_bytes must be >= 0")
        if not math.isfinite(self.compression_ratio) or self.compression_ratio <= 0.0:
            raise ValueError("compression_ratio must be finite and > 0")
        has_reason = bool(self.fallback_reason and self.fallback_reason.strip())
        if self.fallback_used and not has_reason:
            raise ValueError("fallback_reason is required when fallback_used is true")
        if not self.fallback_used and self.fallback_reason is not None:
            raise ValueError("fallback_reason must be None when fallback_used is false")
        object.__setattr__(self, "details", MappingProxyType(dict(self.details)))


class ExecutionCounterSnapshot(NamedTuple):
    run_calls: int
    completed_runs: int
    failed_runs: int
    wait_calls: int
    query_calls: int


class ExecutionCounters:
    """Five plain integers shared by an executor and the work it returns.

    Best-effort diagnostics: increments are not synchronised across threads.
    """

    __slots__ = ("_n",)
    _RUN, _DONE, _FAIL, _WAIT, _QUERY = range(5)

    def __init__(self) -> None:
        self._n = [0, 0, 0, 0, 0]

    def snapshot(self) -> ExecutionCounterSnapshot:
        return ExecutionCounterSnapshot(*self._n)

    def _record_run(self) -> None:
        self._n[self._RUN] += 1

    def _record_completed(self) -> None:
        self._n[self._DONE] += 1

    def _record_failed(self) -> None:
        self._n[self._FAIL] += 1

    def _record_wait(self) -> None:
        self._n[self._WAIT] += 1

    def _record_query(self) -> None:
        self._n[self._QUERY] += 1
