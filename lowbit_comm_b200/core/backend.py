"""What a backend tells the compiler about itself, and the protocol it implements.

`BackendCapabilities` is the answer to "what can you do for this compile context?"; the compiler turns a
mismatch into a rejection reason (`BackendCapabilities.why_not`).  `StrategyChoice` is the answer of an
automatic strategy selector, with the evidence it rests on.  Field names follow the reference
(ccdl_comm/backend.py:15-116).
"""

from __future__ import annotations

from collections.abc import Callable, Mapping
from dataclasses import dataclass, field
from typing import Protocol, runtime_checkable

from ._checks import freeze, is_plain_int, need_text, need_texts, read_only, text_set, text_tuple
from .plan import CommunicationPlan, CompileContext


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
        bits = frozenset(self.bits)
        if any(not is_plain_int(b) or b <= 0 for b in bits):
            raise ValueError("bits must contain positive integers")
        freeze(self, bits=bits, warnings=text_tuple(self.warnings, "warnings"), details=read_only(self.details),
               **{name: text_set(getattr(self, name), name)
                  for name in ("collectives", "strategies", "dtypes", "output_layouts", "features")})
        if not self.available and not (self.reason and self.reason.strip()):
            raise ValueError("reason is required when backend is unavailable")

    def why_not(self, plan: CommunicationPlan, context: CompileContext, *,
                normalize_dtype: Callable[[str], str] = str) -> str | None:
        """The first reason this backend cannot serve `plan` in `context`, or None when it can.  The compiler
        collects these reasons for every candidate it had to pass over."""

        if not self.available:
            return self.reason or "backend is unavailable"
        bit = None if plan.compression is None else plan.compression.bit
        dtypes = {normalize_dtype(name) for name in self.dtypes}
        checks = (
            (plan.collective in self.collectives, f"collective {plan.collective!r}"),
            (plan.strategy in self.strategies, f"strategy {plan.strategy!r}"),
            (normalize_dtype(context.dtype) in dtypes, f"dtype {context.dtype!r}"),
            (bit is None or bit in self.bits, f"bit {bit}"),
            (plan.output_layout in self.output_layouts, f"output layout {plan.output_layout!r}"),
            (self.supports_async or not plan.async_op, "async execution"),
            (self.supports_dynamic_shape or not context.allow_dynamic_shape, "dynamic shape"),
        )
        return next((f"{what} is unsupported" for served, what in checks if not served), None)


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
        need_texts(self, "strategy", "reason", "policy_id")
        for name in ("expected_speedup", "observed_speedup"):
            speedup = getattr(self, name)
            if speedup is not None and speedup <= 0:
                raise ValueError(f"{name} must be > 0")
        if self.observed_speedup is not None and not self.baseline:
            raise ValueError("observed_speedup requires an explicit baseline")   # a speed-up over what?
        if self.benchmark_matched and not self.evidence:
            raise ValueError("benchmark-matched choices require evidence")
        freeze(self, fallback=text_tuple(self.fallback, "fallback", message="fallback strategies must not be empty"))

    @property
    def speedup(self) -> float | None:
        """The recorded speed-up, whichever kind it is (same-semantics expectation or cross-semantics observation)."""

        return self.expected_speedup if self.expected_speedup is not None else self.observed_speedup

    def explain(self) -> str:
        parts = [f"{self.strategy}: {self.reason} [{self.policy_id}]"]
        if self.speedup is not None:
            against = f" over {self.baseline}" if self.baseline else ""
            parts.append(f"{self.speedup:.2f}x{against}")
        if self.evidence:
            parts.append(f"evidence: {self.evidence}")
        if self.fallback:
            parts.append("then " + ", ".join(self.fallback))
        return "; ".join(parts)


@runtime_checkable
class AutoStrategySelector(Protocol):
    """Backend-owned policy: picks one concrete strategy for an `auto` request without running anything."""

    def __call__(self, plan: CommunicationPlan, context: CompileContext) -> StrategyChoice: ...


@runtime_checkable
class CommunicationBackend(Protocol):
    name: str
    abi_version: int

    def capabilities(self, context: CompileContext) -> BackendCapabilities: ...

    def compile(self, plan: CommunicationPlan, context: CompileContext): ...
