"""Plans, registry, strict strategy resolution, capability rejection, cache keys and the LRU cache."""

from dataclasses import replace

import pytest

from lowbit_comm_b200 import (BackendCapabilities, BackendKey, BackendRegistry, CommunicationPlan, CommunicationStage,
                              CompileCache, CompileContext, CompressionConfig, ExecutionCounters, ExecutionInfo,
                              ImmediateWork, StrategyChoice, UnsupportedCollective, WorkspacePolicy, compile, resolve_plan)
from lowbit_comm_b200.exceptions import BackendRegistrationError

CFG = CompressionConfig()


def info(strategy, backend="fake"):
    return ExecutionInfo(requested_strategy=strategy, executed_strategy=strategy, backend=backend, fallback_used=False,
                         fallback_reason=None, stage_names=("s",), original_bytes=128, compressed_bytes=66,
                         compression_ratio=128 / 66, workspace_cache_hit=False, async_capable=True, fast_path="fake")


class FakeExecutor:
    def __init__(self, strategy, backend="fake"):
        self.execution_info = info(strategy, backend)
        self.execution_counters = ExecutionCounters()
        self.calls = []

    def run(self, tensor, out=None):
        self.calls.append((tensor, out))
        return ImmediateWork(("done", tensor), self.execution_info, self.execution_counters)


class FakeBackend:
    abi_version = 1

    def __init__(self, name="fake", strategies=("all_gather", "reduce_scatter"), available=True, dtypes=("bf16",),
                 bits=(8,), layouts=("full", "shard"), collectives=("all_reduce", "reduce_scatter"), async_ok=True):
        self.name = name
        self._caps = BackendCapabilities(backend=name, available=available, collectives=frozenset(collectives),
                                         strategies=frozenset(strategies), dtypes=frozenset(dtypes),
                                         bits=frozenset(bits), output_layouts=frozenset(layouts),
                                         supports_async=async_ok, reason=None if available else "switched off")
        self.compiled = []

    def capabilities(self, context):
        return self._caps

    def compile(self, plan, context):
        self.compiled.append(plan.strategy)
        return FakeExecutor(plan.strategy, self.name)


def ctx(**kw):
    base = dict(rank=0, world_size=4, device="cuda:0", shape=(1024,), dtype="bf16")
    base.update(kw)
    return CompileContext(**base)


def registry_with(backend, strategies=("all_gather", "reduce_scatter"), collective="all_reduce", layout="full"):
    reg = BackendRegistry()
    for s in strategies:
        reg.register(BackendKey(collective, s, backend.name, layout), lambda: backend)
    return reg


def test_plan_and_context_validation():
    with pytest.raises(ValueError):
        CommunicationPlan(collective="", strategy="x")
    with pytest.raises(ValueError):
        CommunicationPlan(collective="all_reduce", strategy="hierarchical")
    with pytest.raises(TypeError):
        CommunicationPlan(collective="all_reduce", strategy="x", compression="int8")
    with pytest.raises(ValueError):
        CommunicationPlan(collective="all_reduce", strategy="x", root=-1)
    stage = CommunicationStage(name="local", collective="reduce_scatter", strategy="compressed")
    plan = CommunicationPlan(collective="all_reduce", strategy="hierarchical", stages=[stage], fallback=["all_gather"])
    assert plan.stages == (stage,) and plan.fallback == ("all_gather",) and plan.backend == "cuda"
    assert plan.reduce_op == "mean" and plan.async_op and plan.output_layout == "full"
    for bad in (dict(world_size=0), dict(rank=4), dict(shape=(2, -1)), dict(local_rank=2, local_world_size=2),
                dict(node_id=1, node_count=1), dict(workspace_budget_bytes=-1), dict(process_groups={"": 1})):
        with pytest.raises(ValueError):
            ctx(**bad)
    c = ctx(process_groups={"local": object()})
    with pytest.raises(TypeError):
        c.process_groups["x"] = 1
    assert c.numel == 1024
    with pytest.raises(ValueError):
        WorkspacePolicy(max_entries=0)


def test_registry_contract():
    backend = FakeBackend()
    reg = registry_with(backend)
    key = BackendKey("all_reduce", "all_gather", "fake", "full")
    assert key in reg and str(key) == "all_reduce:all_gather:fake:full" and reg.resolve(key) is backend
    with pytest.raises(BackendRegistrationError):
        reg.register(key, lambda: backend)
    with pytest.raises(UnsupportedCollective):
        reg.resolve(BackendKey("all_reduce", "tree", "fake", "full"))
    with pytest.raises(TypeError):
        reg.register(("all_reduce",), lambda: backend)
    bad = BackendRegistry()
    bad.register(key, lambda: object())
    with pytest.raises(BackendRegistrationError):
        bad.resolve(key)
    reg.register_strategy_selector("fake", lambda p, c: None)
    with pytest.raises(BackendRegistrationError):
        reg.register_strategy_selector("fake", lambda p, c: None)


def test_compile_requested_strategy_and_run():
    backend = FakeBackend()
    reg = registry_with(backend)
    plan = CommunicationPlan(collective="all_reduce", strategy="reduce_scatter", backend="fake", compression=CFG)
    compiled = compile(plan, ctx(), registry=reg)
    assert compiled.execution_info.executed_strategy == "reduce_scatter" and not compiled.execution_info.fallback_used
    assert compiled.executor.execution_info is compiled.execution_info
    work = compiled.run("t")
    assert work.wait() == ("done", "t") and work.query()
    with pytest.raises(TypeError):
        compiled.run("t", out="o")  # only reduce_scatter/shard plans accept a caller-owned output


def test_explicit_fallback_and_rejection_reasons():
    backend = FakeBackend(strategies=("all_gather",))
    reg = registry_with(backend)
    plan = CommunicationPlan(collective="all_reduce", strategy="reduce_scatter", backend="fake", compression=CFG,
                             fallback=("all_gather",))
    compiled = compile(plan, ctx(), registry=reg)
    assert compiled.execution_info.fallback_used and "explicit fallback" in compiled.execution_info.fallback_reason
    assert compiled.execution_info.requested_strategy == "reduce_scatter"
    with pytest.raises(UnsupportedCollective) as err:
        compile(replace(plan, fallback=()), ctx(), registry=reg)
    assert "strategy 'reduce_scatter' is unsupported" in str(err.value)
    for context, needle in ((ctx(dtype="fp32"), "dtype"), (ctx(allow_dynamic_shape=True), "dynamic shape")):
        with pytest.raises(UnsupportedCollective) as err:
            compile(replace(plan, strategy="all_gather", fallback=()), context, registry=reg)
        assert needle in str(err.value)
    off = FakeBackend(available=False)
    with pytest.raises(UnsupportedCollective) as err:
        compile(replace(plan, strategy="all_gather", fallback=()), ctx(), registry=registry_with(off))
    assert "switched off" in str(err.value)
    four_bit = replace(plan, strategy="all_gather", fallback=(), compression=CompressionConfig(bit=4, allow_experimental=True))
    with pytest.raises(UnsupportedCollective) as err:
        compile(four_bit, ctx(), registry=reg)
    assert "bit 4" in str(err.value)


def test_auto_uses_priority_then_selector():
    backend = FakeBackend()
    reg = registry_with(backend)
    plan = CommunicationPlan(collective="all_reduce", strategy="auto", backend="fake", compression=CFG)
    assert compile(plan, ctx(world_size=2), registry=reg).execution_info.executed_strategy == "all_gather"
    assert compile(plan, ctx(world_size=8), registry=reg).execution_info.executed_strategy == "reduce_scatter"
    assert resolve_plan(plan, ctx(world_size=8), reg).executed_strategy == "reduce_scatter"
    reg.register_strategy_selector("fake", lambda p, c: StrategyChoice(
        strategy="tree", reason="measured", policy_id="p1", benchmark_matched=True, evidence="profiles/x.md",
        expected_speedup=1.5, fallback=("all_gather",)))
    compiled = compile(plan, ctx(world_size=8), registry=reg)
    info_ = compiled.execution_info
    assert info_.executed_strategy == "all_gather" and info_.fallback_used and "tree" in info_.fallback_reason
    assert info_.details["strategy_policy_id"] == "p1" and info_.details["strategy_evidence"] == "profiles/x.md"
    assert compiled.cache_key.strategy_policy_id == "p1"


def test_compile_cache_lru_and_key_identity():
    backend = FakeBackend()
    reg = registry_with(backend)
    cache = CompileCache(max_entries=2)
    plan = CommunicationPlan(collective="all_reduce", strategy="all_gather", backend="fake", compression=CFG)
    a = compile(plan, ctx(), registry=reg, cache=cache)
    assert compile(plan, ctx(), registry=reg, cache=cache) is a and backend.compiled == ["all_gather"]
    b = compile(plan, ctx(shape=(2048,)), registry=reg, cache=cache)
    compile(plan, ctx(), registry=reg, cache=cache)            # refresh a
    compile(plan, ctx(shape=(4096,)), registry=reg, cache=cache)  # evicts b
    assert len(cache) == 2 and cache.get(b.cache_key) is None and cache.get(a.cache_key) is a
    other_group = compile(plan, ctx(process_group=object()), registry=reg)
    assert other_group.cache_key != a.cache_key
    with pytest.raises(ValueError):
        CompileCache(max_entries=0)
    with pytest.raises(TypeError):
        cache.get("key")


def test_backend_contract_violations_are_reported():
    class Liar(FakeBackend):
        def compile(self, plan, context):
            return FakeExecutor("something_else", self.name)

    plan = CommunicationPlan(collective="all_reduce", strategy="all_gather", backend="fake", compression=CFG)
    with pytest.raises(BackendRegistrationError):
        compile(plan, ctx(), registry=registry_with(Liar()))

    class NoExecutor(FakeBackend):
        def compile(self, plan, context):
            return object()

    with pytest.raises(BackendRegistrationError):
        compile(plan, ctx(), registry=registry_with(NoExecutor()))
    with pytest.raises(ValueError):
        BackendCapabilities(backend="x", available=False)
    with pytest.raises(ValueError):
        StrategyChoice(strategy="a", reason="b", policy_id="c", benchmark_matched=True)
    with pytest.raises(ValueError):
        StrategyChoice(strategy="a", reason="b", policy_id="c", benchmark_matched=False, observed_speedup=2.0)


def plan_for(strategy, **kw):
    return CommunicationPlan(collective="all_reduce", strategy=strategy, backend="fake", compression=CFG, **kw)


def test_resolve_plan_is_a_dry_run_over_registry_membership():
    backend = FakeBackend()
    reg = registry_with(backend, strategies=("all_gather", "reduce_scatter"))
    assert resolve_plan(plan_for("all_gather"), ctx(), reg).executed_strategy == "all_gather"
    fell = resolve_plan(plan_for("ring", fallback=("auto", "reduce_scatter")), ctx(), reg)
    assert (fell.executed_strategy, fell.fallback_used) == ("reduce_scatter", True) and "ring" in fell.fallback_reason
    with pytest.raises(UnsupportedCollective, match="no fallback was declared"):
        resolve_plan(plan_for("ring"), ctx(), reg)
    with pytest.raises(UnsupportedCollective, match="no supported fallback"):
        resolve_plan(plan_for("ring", fallback=("tree",)), ctx(), reg)
    declared = resolve_plan(plan_for("auto", fallback=("all_gather",)), ctx(), reg)
    assert declared.requested_strategy == "auto" and declared.executed_strategy == "all_gather" and declared.fallback_used
    generic = resolve_plan(plan_for("auto"), ctx(), reg)                # no selector: the generic order, 4 ranks
    assert generic.executed_strategy == "reduce_scatter" and not generic.fallback_used
    two = resolve_plan(plan_for("auto"), ctx(world_size=2), reg)
    assert two.executed_strategy == "all_gather"
    with pytest.raises(UnsupportedCollective, match="found no registered backend"):
        resolve_plan(plan_for("auto"), ctx(), BackendRegistry())
    reg.register_strategy_selector("fake", lambda plan, context: StrategyChoice(
        "tree", "measured", "policy-1", False, fallback=("all_gather",)))
    chosen = resolve_plan(plan_for("auto"), ctx(), reg)
    assert chosen.executed_strategy == "all_gather" and chosen.fallback_used and chosen.strategy_policy_id == "policy-1"
    lonely = registry_with(backend, strategies=("reduce_scatter",))
    lonely.register_strategy_selector("fake", lambda plan, context: StrategyChoice("tree", "measured", "p", False))
    with pytest.raises(UnsupportedCollective, match="declared fallbacks are not registered"):
        resolve_plan(plan_for("auto"), ctx(), lonely)
    assert backend.compiled == []                                       # nothing was compiled along the way
    for bad in ((None, ctx(), reg), (plan_for("auto"), None, reg), (plan_for("auto"), ctx(), None)):
        with pytest.raises(TypeError):
            resolve_plan(*bad)


def test_backends_that_break_the_contract_are_reported_as_such():
    def compile_with(backend, strategy="all_gather"):
        reg = BackendRegistry()
        reg.register(BackendKey("all_reduce", strategy, "fake", "full"), lambda: backend)
        return compile(plan_for(strategy), ctx(), registry=reg)

    misnamed = FakeBackend(name="other")
    with pytest.raises(BackendRegistrationError, match="does not match registry key"):
        compile_with(misnamed)

    class NoCaps(FakeBackend):
        def capabilities(self, context):
            return {"available": True}

    with pytest.raises(BackendRegistrationError, match="did not return BackendCapabilities"):
        compile_with(NoCaps())

    class ForeignCaps(FakeBackend):
        def capabilities(self, context):
            return replace(self._caps, backend="elsewhere")

    with pytest.raises(BackendRegistrationError, match="capability backend"):
        compile_with(ForeignCaps())

    class NoExecutor(FakeBackend):
        def compile(self, plan, context):
            return object()

    with pytest.raises(BackendRegistrationError, match="did not return a CompiledExecutor"):
        compile_with(NoExecutor())

    class BadInfo(FakeBackend):
        def compile(self, plan, context):
            executor = FakeExecutor(plan.strategy)
            executor.execution_info = "fast"
            return executor

    with pytest.raises(BackendRegistrationError, match="did not expose ExecutionInfo"):
        compile_with(BadInfo())

    class OtherBackendInfo(FakeBackend):
        def compile(self, plan, context):
            return FakeExecutor(plan.strategy, backend="elsewhere")

    with pytest.raises(BackendRegistrationError, match="inconsistent backend"):
        compile_with(OtherBackendInfo())

    class OtherStrategyInfo(FakeBackend):
        def compile(self, plan, context):
            return FakeExecutor("ring")

    with pytest.raises(BackendRegistrationError, match="inconsistent executed strategy"):
        compile_with(OtherStrategyInfo())

    class FrozenExecutor:
        __slots__ = ("_info",)

        def __init__(self, strategy):
            self._info = info(strategy)

        execution_info = property(lambda self: self._info)

        def run(self, tensor):
            return ImmediateWork(tensor)

    class Frozen(FakeBackend):
        def compile(self, plan, context):
            return FrozenExecutor(plan.strategy)

    with pytest.raises(BackendRegistrationError, match="must allow compile-time ExecutionInfo binding"):
        compile_with(Frozen())

    reg = registry_with(FakeBackend())
    reg.register_strategy_selector("fake", lambda plan, context: "all_gather")
    with pytest.raises(BackendRegistrationError, match="did not return StrategyChoice"):
        compile(plan_for("auto"), ctx(), registry=reg)
    with pytest.raises(TypeError, match="CompileCache"):
        compile(plan_for("all_gather"), ctx(), registry=registry_with(FakeBackend()), cache={})


def test_compile_cache_checks_what_goes_in():
    cache = CompileCache(max_entries=2)
    compiled = compile(plan_for("all_gather"), ctx(), registry=registry_with(FakeBackend()), cache=cache)
    assert cache.max_entries == 2 and len(cache) == 1 and cache.get(compiled.cache_key) is compiled
    cache.put(compiled.cache_key, compiled)
    with pytest.raises(TypeError):
        cache.put("key", compiled)
    with pytest.raises(TypeError):
        cache.put(compiled.cache_key, "compiled")
    with pytest.raises(TypeError):
        cache.get_or_create(compiled.cache_key, "factory")
    cache.clear()
    with pytest.raises(TypeError, match="must return"):
        cache.get_or_create(compiled.cache_key, lambda: "not a plan")
    assert len(cache) == 0
    with pytest.raises(ValueError):
        CompileCache(max_entries=0)
