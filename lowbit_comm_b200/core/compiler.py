"""Compile-once control plane: plan + context -> compiled executor.

Parity: ccdl_comm/compiler.py:117-626 (`compile`, `resolve_plan`,
`CompileCache`, candidate ordering, capability rejection, cache key).  All
strategy, fallback and capability decisions are taken here so that
`CompiledCommunicationPlan.run` does none of them.
"""

from __future__ import annotations

import threading
from collections import OrderedDict
from collections.abc import Callable, Iterable
from dataclasses import dataclass, replace

from ..exceptions import BackendRegistrationError, UnsupportedCollective
from .backend import BackendCapabilities, StrategyChoice
from .executor import CompileCacheKey, CompiledCommunicationPlan, CompiledExecutor
from .info import ExecutionInfo
from .plan import CommunicationPlan, CompileContext
from .registry import BackendKey, BackendRegistry

_DTYPE_ALIASES = {"float16": "fp16", "half": "fp16", "bfloat16": "bf16", "float32": "fp32", "float": "fp32"}


def normalize_dtype(name: str) -> str:
    text = name.strip().lower().removeprefix("torch.")
    return _DTYPE_ALIASES.get(text, text)


@dataclass(frozen=True)
class ResolvedPlan:
    requested_strategy: str
    executed_strategy: str
    fallback_used: bool
    fallback_reason: str | None
    selection_reason: str | None = None
    strategy_policy_id: str | None = None
    benchmark_matched: bool = False
    strategy_evidence: str | None = None
    expected_speedup: float | None = None
    observed_speedup: float | None = None
    comparison_baseline: str | None = None


class CompileCache:
    """Thread-safe LRU of compiled plans (default 128 entries)."""

    def __init__(self, *, max_entries: int = 128) -> None:
        if isinstance(max_entries, bool) or not isinstance(max_entries, int) or max_entries <= 0:
            raise ValueError("max_entries must be a positive integer")
        self._cap = max_entries
        self._items: OrderedDict[CompileCacheKey, CompiledCommunicationPlan] = OrderedDict()
        self._guard = threading.RLock()

    @property
    def max_entries(self) -> int:
        return self._cap

    @staticmethod
    def _need_key(key: object) -> None:
        if not isinstance(key, CompileCacheKey):
            raise TypeError("key must be a CompileCacheKey")

    def _store(self, key: CompileCacheKey, value: CompiledCommunicationPlan) -> None:
        self._items[key] = value
        self._items.move_to_end(key)
        while len(self._items) > self._cap:
            self._items.popitem(last=False)

    def get(self, key: CompileCacheKey) -> CompiledCommunicationPlan | None:
        self._need_key(key)
        with self._guard:
            hit = self._items.get(key)
            if hit is not None:
                self._items.move_to_end(key)
            return hit

    def put(self, key: CompileCacheKey, compiled: CompiledCommunicationPlan) -> None:
        self._need_key(key)
        if not isinstance(compiled, CompiledCommunicationPlan):
            raise TypeError("compiled must be a CompiledCommunicationPlan")
        with self._guard:
            self._store(key, compiled)

    def get_or_create(self, key: CompileCacheKey,
                      factory: Callable[[], CompiledCommunicationPlan]) -> CompiledCommunicationPlan:
        self._need_key(key)
        if not callable(factory):
            raise TypeError("factory must be callable")
        with self._guard:
            hit = self._items.get(key)
            if hit is not None:
                self._items.move_to_end(key)
                return hit
            made = factory()
            if not isinstance(made, CompiledCommunicationPlan):
                raise TypeError("factory must return a CompiledCommunicationPlan")
            self._store(key, made)
            return made

    def clear(self) -> None:
        with self._guard:
            self._items.clear()

    def __len__(self) -> int:
        with self._guard:
            return len(self._items)


_DEFAULT_REGISTRY = BackendRegistry()


def default_registry() -> BackendRegistry:
    return _DEFAULT_REGISTRY


def auto_priority(context: CompileContext) -> tuple[str, ...]:
    """Generic ordering used when a backend registered no selector."""

    if context.world_size <= 2:
        return ("all_gather", "all_reduce", "topology", "ring", "reduce_scatter", "hierarchical")
    if (context.node_count or 1) > 1 and context.process_groups:
        return ("hierarchical", "reduce_scatter", "all_gather", "topology", "all_reduce", "ring")
    return ("reduce_scatter", "hierarchical", "all_gather", "topology", "all_reduce", "ring")


def _key(plan: CommunicationPlan, strategy: str) -> BackendKey:
    return BackendKey.checked(plan.collective, strategy, plan.backend, plan.output_layout)


def _dedupe(pairs: Iterable[tuple[str, str]]) -> tuple[tuple[str, str], ...]:
    seen: dict[str, str] = {}
    for strategy, origin in pairs:
        seen.setdefault(strategy, origin)
    return tuple(seen.items())


def _selector_choice(plan: CommunicationPlan, context: CompileContext,
                     registry: BackendRegistry) -> StrategyChoice | None:
    if plan.strategy != "auto":
        return None
    selector = registry.strategy_selector(plan.backend)
    if selector is None:
        return None
    choice = selector(plan, context)
    if not isinstance(choice, StrategyChoice):
        raise BackendRegistrationError(
            f"strategy selector for backend {plan.backend!r} did not return StrategyChoice")
    return choice


def _candidates(plan: CommunicationPlan, context: CompileContext, registry: BackendRegistry,
                choice: StrategyChoice | None) -> tuple[tuple[str, str], ...]:
    declared = [(s, "explicit") for s in plan.fallback if s != "auto"]
    if plan.strategy != "auto":
        return _dedupe([(plan.strategy, "requested"), *declared])
    if choice is not None:
        return _dedupe([(choice.strategy, "auto"),
                        *((s, "auto_fallback") for s in choice.fallback), *declared])
    preferred = auto_priority(context)
    registered = registry.strategies_for(plan.collective, plan.backend, plan.output_layout)
    extra = sorted(registered - {"auto", *plan.fallback, *preferred})
    return _dedupe([*declared, *((s, "auto") for s in (*preferred, *extra))])


def _describe(plan: CommunicationPlan, context: CompileContext, strategy: str, origin: str,
              choice: StrategyChoice | None) -> ResolvedPlan:
    if origin == "requested":
        return ResolvedPlan(plan.strategy, strategy, False, None)
    if origin == "explicit" and plan.strategy != "auto":
        return ResolvedPlan(plan.strategy, strategy, True,
                            f"explicit fallback from {plan.strategy} to {strategy}")
    if choice is not None:
        fell_back = strategy != choice.strategy
        why = f"auto fallback from selected strategy {choice.strategy} to {strategy}" if fell_back else None
        return ResolvedPlan("auto", strategy, fell_back, why,
                            selection_reason=choice.reason, strategy_policy_id=choice.policy_id,
                            benchmark_matched=choice.benchmark_matched, strategy_evidence=choice.evidence,
                            expected_speedup=choice.expected_speedup, observed_speedup=choice.observed_speedup,
                            comparison_baseline=choice.baseline)
    first = auto_priority(context)[0]
    fell_back = strategy != first
    why = f"auto fallback from unavailable preferred strategy {first} to {strategy}" if fell_back else None
    return ResolvedPlan("auto", strategy, fell_back, why)


def capability_rejection(caps: BackendCapabilities, plan: CommunicationPlan,
                         context: CompileContext) -> str | None:
    """Reason the backend cannot serve `plan`, or None when it can (dtype spellings are normalised first)."""

    return caps.why_not(plan, context, normalize_dtype=normalize_dtype)


def _pick_backend(plan: CommunicationPlan, context: CompileContext, registry: BackendRegistry):
    choice = _selector_choice(plan, context, registry)
    refused: list[str] = []
    for strategy, origin in _candidates(plan, context, registry, choice):
        key = _key(plan, strategy)
        if key not in registry:
            close = ", ".join(str(k) for k in registry.nearest(key, limit=2))
            refused.append(f"{strategy}: backend key is not registered" + (f" (closest: {close})" if close else ""))
            continue
        backend = registry.resolve(key)
        if backend.name != plan.backend:
            raise BackendRegistrationError(f"backend name {backend.name!r} does not match registry key {key}")
        caps = backend.capabilities(context)
        if not isinstance(caps, BackendCapabilities):
            raise BackendRegistrationError(f"backend for {key} did not return BackendCapabilities")
        if caps.backend != plan.backend:
            raise BackendRegistrationError(
                f"capability backend {caps.backend!r} does not match registry key {key}")
        effective = replace(plan, strategy=strategy, fallback=())
        why_not = capability_rejection(caps, effective, context)
        if why_not is not None:
            refused.append(f"{strategy}: {why_not}")
            continue
        resolved = _describe(plan, context, strategy, origin, choice)
        if plan.strategy == "auto" and resolved.fallback_used and refused:
            resolved = replace(resolved, fallback_reason=(
                f"{resolved.fallback_reason}; rejected candidates: " + "; ".join(refused)))
        return resolved, effective, backend
    reason = "no registered backend supports the requested compile context"
    if refused:
        reason += "; " + "; ".join(refused)
    raise UnsupportedCollective(f"{plan.collective}:{plan.strategy}", reason=reason)


def make_cache_key(requested: CommunicationPlan, effective: CommunicationPlan, context: CompileContext,
                   registry: BackendRegistry, resolved: ResolvedPlan) -> CompileCacheKey:
    return CompileCacheKey.of(requested, effective, context, registry, resolved.strategy_policy_id)


def _build(backend, effective: CommunicationPlan, context: CompileContext, resolved: ResolvedPlan,
           cache_key: CompileCacheKey) -> CompiledCommunicationPlan:
    key = _key(effective, effective.strategy)
    executor = backend.compile(effective, context)
    if not isinstance(executor, CompiledExecutor):
        raise BackendRegistrationError(f"backend for {key} did not return a CompiledExecutor")
    info = executor.execution_info
    if not isinstance(info, ExecutionInfo):
        raise BackendRegistrationError(f"executor for {key} did not expose ExecutionInfo")
    if info.backend != effective.backend:
        raise BackendRegistrationError(f"executor for {key} reported inconsistent backend {info.backend!r}")
    if info.executed_strategy != effective.strategy:
        raise BackendRegistrationError(
            f"executor for {key} reported inconsistent executed strategy {info.executed_strategy!r}")
    details = dict(info.details)
    if resolved.selection_reason is not None:
        details.update(
            strategy_selection_reason=resolved.selection_reason,
            strategy_policy_id=resolved.strategy_policy_id,
            strategy_benchmark_matched=resolved.benchmark_matched,
            strategy_evidence=resolved.strategy_evidence,
            strategy_expected_speedup=resolved.expected_speedup,
            strategy_observed_speedup=resolved.observed_speedup,
            strategy_comparison_baseline=resolved.comparison_baseline,
        )
    bound = replace(info, requested_strategy=resolved.requested_strategy,
                    executed_strategy=resolved.executed_strategy, fallback_used=resolved.fallback_used,
                    fallback_reason=resolved.fallback_reason, details=details)
    try:
        executor.execution_info = bound
    except (AttributeError, TypeError) as exc:
        raise BackendRegistrationError(
            f"executor for {key} must allow compile-time ExecutionInfo binding") from exc
    if executor.execution_info is not bound:
        raise BackendRegistrationError(f"executor for {key} did not retain bound ExecutionInfo")
    return CompiledCommunicationPlan(executor=executor, execution_info=bound, cache_key=cache_key)


def compile(plan: CommunicationPlan, context: CompileContext, *, registry: BackendRegistry | None = None,
            cache: CompileCache | None = None) -> CompiledCommunicationPlan:
    """Resolve strategy and backend once and return a reusable compiled plan."""

    reg = _DEFAULT_REGISTRY if registry is None else registry
    if cache is not None and not isinstance(cache, CompileCache):
        raise TypeError("cache must be a CompileCache or None")
    resolved, effective, backend = _pick_backend(plan, context, reg)
    cache_key = make_cache_key(plan, effective, context, reg, resolved)
    build = lambda: _build(backend, effective, context, resolved, cache_key)  # noqa: E731
    return build() if cache is None else cache.get_or_create(cache_key, build)


def resolve_plan(plan: CommunicationPlan, context: CompileContext, registry: BackendRegistry) -> ResolvedPlan:
    """Dry run of strategy resolution using only registry membership."""

    if not isinstance(plan, CommunicationPlan):
        raise TypeError("plan must be a CommunicationPlan")
    if not isinstance(context, CompileContext):
        raise TypeError("context must be a CompileContext")
    if not isinstance(registry, BackendRegistry):
        raise TypeError("registry must be a BackendRegistry")
    if plan.strategy != "auto":
        if _key(plan, plan.strategy) in registry:
            return ResolvedPlan(plan.strategy, plan.strategy, False, None)
        for alt in plan.fallback:
            if alt != "auto" and _key(plan, alt) in registry:
                return ResolvedPlan(plan.strategy, alt, True, f"explicit fallback from {plan.strategy} to {alt}")
        tail = "no supported fallback was declared" if plan.fallback else "no fallback was declared"
        raise UnsupportedCollective(f"{plan.collective}:{plan.strategy}",
                                    reason=f"explicit strategy unavailable and {tail}")
    for alt in plan.fallback:
        if alt != "auto" and _key(plan, alt) in registry:
            return ResolvedPlan("auto", alt, True, f"explicit fallback from auto to {alt}")
    registered = registry.strategies_for(plan.collective, plan.backend, plan.output_layout) - {"auto"}
    if not registered:
        raise UnsupportedCollective(f"{plan.collective}:auto",
                                    reason="auto strategy found no registered backend for the requested dimensions")
    choice = _selector_choice(plan, context, registry)
    if choice is not None:
        for name in (choice.strategy, *choice.fallback, *plan.fallback):
            if name != "auto" and name in registered:
                return _describe(plan, context, name, "auto", choice)
        raise UnsupportedCollective(
            f"{plan.collective}:auto",
            reason=f"selected strategy {choice.strategy!r} and its declared fallbacks are not registered")
    preferred = auto_priority(context)
    order = (*preferred, *sorted(registered.difference(preferred)))
    picked = next(s for s in order if s in registered)
    return _describe(plan, context, picked, "auto", None)
