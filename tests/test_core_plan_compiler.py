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
