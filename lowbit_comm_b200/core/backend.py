"""Backend capability records and the backend protocol.

Parity: ccdl_comm/backend.py:15-116.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Protocol, runtime_checkable

from ._checks import is_plain_int, need_text
from .plan import CommunicationPlan, CompileContext

_STRING_SETS = ("collectives", "strategies", "dtypes", "output_layouts", "features")


@dataclass(frozen=True)
class BackendCapabilities:
    """What one backend can do for one compile context."""

    backend: str
    available: bool
    collectives: frozenset[str] = frozenset()
    strategies: frozenset[str] = frozenset()
    dtypes: frozenset[str] = frozenset()
    bits: frozenset[int] = frozenset()
    output_layouts: frozenset[str] = frozenset()
    supports_async: bool = False
    supports_dynamic_shape: bool = False
    features: frozenset[str] = frozenset()
    reason: str | None = None
    warnings: tuple[str, ...] = ()
    details: Mapping[str, object] = field(default_factory=dict)

    def __post_init__(self) -> None:
        need_text(self.backend, "backend")
        for attr in _STRING_SETS:
            values = frozenset(getattr(self, attr))
            if any(not isinstance(v, str) or not v.strip() for v in values):
                raise ValueError(f"{attr} must contain non-empty strings")
            object.__setattr__(self, attr, values)
        bits = frozenset(self.bits)
        if any(not is_plain_int(b) or b <= 0 for b in bits):
            raise ValueError("bits must contain positive integers")
        object.__setattr__(self, "bits", bits)
        notes = tuple(self.warnings)
        if any(not isinstance(w, str) or not w.strip() for w in notes):
            raise ValueError("warnings must contain non-empty strings")
        object.__setattr__(self, "warnings", notes)
        object.__setattr__(self, "details", MappingProxyType(dict(self.details)))
        if not self.available and not (self.reason and self.reason.strip()):
            raise ValueError("reason is required when backend is unavailable")


@dataclass(frozen=True)
class StrategyChoice:
    """An explainable automatic strategy decision."""

    strategy: str
    reason: str
    policy_id: str
    benchmark_matched: bool
    expected_speedup: float | None = None
    observed_speedup: float | None = None
    baseline: str | None = None
    evidence: str | None = None
    fallback: tuple[str, ...] = ()

    def __post_init__(self) -> None:
        for attr in ("strategy", "reason", "policy_id"):
            need_text(getattr(self, attr), attr)
        for attr in ("expected_speedup", "observed_speedup"):
            value = getattr(self, attr)
            if value is not None and value <= 0:
                raise ValueError(f"{attr} must be > 0")
        if self.observed_speedup is not None and not self.baseline:
            raise ValueError("observed_speedup requires an explicit baseline")
        if self.benchmark_matched and not self.evidence:
            raise ValueError("benchmark-matched choices require evidence")
        names = tuple(self.fallback)
        if any(not n.strip() for n in names):
            raise ValueError("fallback strategies must not be empty")
        object.__setattr__(self, "fallback", names)


@runtime_checkable
class AutoStrategySelector(Protocol):
    def __call__(self, plan: CommunicationPlan, context: CompileContext) -> StrategyChoice: ...


@runtime_checkable
class CommunicationBackend(Protocol):
    name: str
    abi_version: int

    def capabilities(self, context: CompileContext) -> BackendCapabilities: ...

    def compile(self, plan: CommunicationPlan, context: CompileContext): ...
