"""Behaviour the control plane adds on top of the reference's surface: write-once registry with diagnostics,
grouped cache key, settle-once work objects, route lists, device wait status, named compression profiles."""

import pytest

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.core.backend import BackendCapabilities
from lowbit_comm_b200.core.executor import CompileCacheKey
from lowbit_comm_b200.core.info import ExecutionCounters
from lowbit_comm_b200.core.plan import CommunicationPlan, CompileContext
from lowbit_comm_b200.core.registry import BackendKey, BackendRegistry
from lowbit_comm_b200.core.work import BoundCollectiveWork, CompletionWork, ImmediateWork, bind_execution_work
from lowbit_comm_b200.exceptions import (AsyncCommunicationError, BackendRegistrationError, DeviceWaitStatus,
                                         UnsupportedCollective)
from lowbit_comm_b200.parallel.bucket_fusion import BucketDescriptor, plan_bucket_fusion
from lowbit_comm_b200.parallel.collectives._routes import as_requested, first_that_serves, injected
from lowbit_comm_b200.parallel.strategy_table import CudaStrategyRule, CudaStrategyTable, PRODUCTION_PROFILE


class _Backend:
    name, abi_version = "fake", 1

    def capabilities(self, context):
        return BackendCapabilities(backend="fake", available=True)

    def compile(self, plan, context):
        raise NotImplementedError


def test_registry_is_write_once_and_suggests_near_keys():
    registry = BackendRegistry()

    @registry.provides(collective="all_reduce", strategy="compressed", backend="cuda", output_layout="full")
    class Provided(_Backend):
        pass

    key = BackendKey("all_reduce", "compressed", "cuda", "full")
    assert key in registry and isinstance(registry.resolve(key), Provided)
    with pytest.raises(BackendRegistrationError, match="already registered"):
        registry.register(key, _Backend)
    with pytest.raises(ValueError):
        registry.register(BackendKey("all_reduce", " ", "cuda", "full"), _Backend)
    with pytest.raises(TypeError):
        registry.register(key._replace(strategy="other"), "not callable")
    typo = key._replace(strategy="compresed")
    assert typo.distance(key) == 1 and registry.nearest(typo) == (key,)
    assert registry.nearest(BackendKey("a", "b", "c", "d")) == ()
    assert registry.strategies_for("all_reduce", "cuda", "full") == {"compressed"}
    with pytest.raises(UnsupportedCollective):
        registry.resolve(typo)
    registry.register(typo, lambda: object())
    with pytest.raises(BackendRegistrationError, match="did not return"):
        registry.resolve(typo)
    registry.register_strategy_selector("cuda", lambda plan, context: None)
    with pytest.raises(BackendRegistrationError):
        registry.register_strategy_selector("cuda", lambda plan, context: None)
    assert registry.strategy_selector("cuda") is not None and registry.strategy_selector("other") is None


def test_cache_key_groups_facts_and_names_what_changed():
    plan = CommunicationPlan(collective="all_reduce", strategy="compressed", backend="cuda", output_layout="full",
                             compression=CompressionConfig())
    ctx = CompileContext(rank=0, world_size=4, device="cuda:0", shape=(1024,), dtype="bf16")
    registry = BackendRegistry()
    one = CompileCacheKey.of(plan, plan, ctx, registry, None)
    same = CompileCacheKey.of(plan, plan, ctx, registry, None)
    assert one == same and hash(one) == hash(same) and one.differs_from(same) == ()
    assert (one.collective, one.bit, one.group_size, one.world_size, one.shape_class) == ("all_reduce", 8, 64, 4, (1024,))
    other_ctx = CompileContext(rank=1, world_size=4, device="cuda:1", shape=(2048,), dtype="bf16")
    moved = CompileCacheKey.of(plan, plan, other_ctx, BackendRegistry(), None)
    assert set(moved.differs_from(one)) == {"registry_identity", "shape_class", "rank", "device"}
    with pytest.raises(AttributeError):
        one.no_such_fact


def test_work_objects_settle_once_and_count_once():
    counters = ExecutionCounters()
    calls = []
    work = CompletionWork("early", complete=lambda: calls.append(1) or "late", execution_counters=counters)
    assert not work.query() and work.wait() == "late" and work.wait() == "late" and calls == [1]
    snap = counters.snapshot()
    assert (snap.completed_runs, snap.failed_runs, snap.wait_calls, snap.query_calls) == (1, 0, 2, 1)

    def boom():
        raise RuntimeError("transport died")

    failing = CompletionWork(None, complete=boom, execution_counters=counters)
    for _ in range(2):
        with pytest.raises(RuntimeError, match="transport died"):
            failing.wait()
    assert counters.snapshot().failed_runs == 1 and failing.query()

    class Foreign:
        def wait(self):
            return 7

        def is_completed(self):
            return False

    bound = bind_execution_work(Foreign(), None, counters)
    assert isinstance(bound, BoundCollectiveWork) and not bound.query() and bound.wait() == 7 and bound.query()
    plain = bind_execution_work(3, None, counters)
    assert isinstance(plain, ImmediateWork) and plain.result == 3 and plain == ImmediateWork(3)
    assert bind_execution_work(plain, None, counters) is plain
    elsewhere = bind_execution_work(plain, None, ExecutionCounters())
    assert elsewhere is not plain and elsewhere.result == 3


def test_routes_fall_through_on_refusal_only():
    def declines(t):
        raise UnsupportedCollective("x", reason="not here")

    assert first_that_serves([declines, lambda t: t + 1], 1, what="demo") == 2
    with pytest.raises(UnsupportedCollective, match="not here"):
        first_that_serves([declines], 1, what="demo")
    with pytest.raises(UnsupportedCollective, match="no demo route"):
        first_that_serves([], 1, what="demo")
    with pytest.raises(ZeroDivisionError):
        first_that_serves([lambda t: 1 / 0, lambda t: t], 1, what="demo")
    seen = {}
    injected(lambda t, **kw: seen.update(kw), {"op": "sum"}, out=None, extra=5)(0)
    assert seen == {"op": "sum", "extra": 5}
    assert as_requested(4, False) == 4 and as_requested(4, True).wait() == 4
    assert as_requested(ImmediateWork(5), False) == 5


def test_device_wait_status_round_trips_into_the_error():
    quiet = DeviceWaitStatus()
    assert not quiet.timed_out
    status = DeviceWaitStatus(code=1, phase=0, peer=3, seen=4, expected=5)
    error = AsyncCommunicationError.from_wait(2, status)
    assert status.timed_out and "rank 2" in str(error) and "reduce-scatter" in str(error)
    assert error.status == {"code": 1, "phase": 0, "peer": 3, "seen": 4, "expected": 5}
    assert DeviceWaitStatus(1, 7, 0, 0, 0).phase_name == "phase 7"
    assert "peers' quantized rows" in DeviceWaitStatus(1, 9, 0, 0, 0).phase_name
    assert AsyncCommunicationError("plain").status == {}


def test_named_profiles_and_labels():
    assert CompressionConfig.production() == CompressionConfig()
    four = CompressionConfig.int4("e2m1", group_size=32)
    assert (four.bit, four.quant_type, four.group_size, four.max_code) == (4, "e2m1", 32, 7)
    assert four.evolve(topk=1).describe() == "int4 g32 e2m1 top1 ef=always"
    with pytest.raises(ValueError):
        four.evolve(group_size=48)
    assert CompressionConfig.from_dict({**four.to_dict(), "from_the_future": 1}) == four


def test_fusion_plan_counts_saved_launches():
    buckets = [BucketDescriptor(i, 100, "bf16") for i in range(5)] + [BucketDescriptor(5, 100, "bf16", requires_full_bucket=True)]
    plan = plan_bucket_fusion(buckets, max_bucket_count=3)
    assert [g.bucket_indices for g in plan.groups] == [(0, 1, 2), (3, 4), (5,)]
    assert plan.launches_saved == 3 and plan.to_metadata()["fused_bucket_count"] == 5
    assert plan_bucket_fusion(buckets, enabled=False).launches_saved == 0


def test_strategy_table_lookup_is_by_domain_and_rejects_overlap():
    table = CudaStrategyTable.for_b200()
    plan = CommunicationPlan(collective="all_reduce", strategy="auto", backend="cuda", output_layout="full",
                             compression=CompressionConfig(error_feedback=False))
    big = CompileContext(rank=0, world_size=8, device="cuda:0", shape=(1 << 26,), dtype="bf16", device_architecture="sm_100")
    rule = table.lookup(plan, big)
    assert rule is not None and rule.strategy == "reduce_scatter" and table.select(plan, big).benchmark_matched
    small = CompileContext(rank=0, world_size=8, device="cuda:0", shape=(1 << 20,), dtype="bf16", device_architecture="sm_100")
    assert table.lookup(plan, small) is None and table.select(plan, small).strategy == "native_nccl"
    pair = CompileContext(rank=0, world_size=2, device="cuda:0", shape=(1 << 20,), dtype="bf16", device_architecture="sm_100")
    assert table.lookup(plan, pair).strategy == "all_gather"
    odd = CompileContext(rank=0, world_size=3, device="cuda:0", shape=(1 << 26,), dtype="bf16", device_architecture="sm_100")
    assert table.lookup(plan, odd) is None and "world_size" in table.select(plan, odd).reason
    base = dict(collective="all_reduce", output_layout="full", device_architecture="sm_100", world_size=2, dtype="bf16",
                compression=PRODUCTION_PROFILE, strategy="all_gather", speedup=1.1, same_semantics_baseline=True)
    with pytest.raises(ValueError, match="overlapping"):
        CudaStrategyTable((CudaStrategyRule(min_numel=0, max_numel=10, **base),
                           CudaStrategyRule(min_numel=10, max_numel=20, **base)))


def test_peer_group_turns_the_status_word_into_an_error():
    from lowbit_comm_b200.parallel.peer_memory import PeerGroup

    class FakeExt:
        word = (0, 0, 0, 0, 0)

        def status_read(self, host):
            return self.word

    group = object.__new__(PeerGroup)       # no arena: only the status path is exercised
    group._ext, group.status_host, group.rank = FakeExt(), 0, 5
    group.check_status()
    assert group.read_status() == {"code": 0, "phase": 0, "peer": 0, "seen": 0, "expected": 0}
    FakeExt.word = (1, 1, 2, 6, 7)
    with pytest.raises(AsyncCommunicationError, match=r"rank 5 \(phase 1: all-gather, flag 2, saw epoch 6, expected 7\)") as info:
        group.check_status()
    assert info.value.status["expected"] == 7 and info.value.status["seen"] == 6


def test_gather_prefetch_switch_rounds_down_to_a_built_depth():
    from lowbit_comm_b200.ops.loader import load_cuda_extension

    status = load_cuda_extension()
    if not status.available:
        pytest.skip(f"extension not built: {status.reason}")
    ext = status.module
    try:
        for asked, got in ((0, 0), (1, 0), (2, 2), (3, 2), (4, 4), (9, 4), (-1, 0)):
            ext.set_gather_prefetch(asked)
            assert ext.get_gather_prefetch() == got
    finally:
        ext.set_gather_prefetch(0)


def test_native_shortcuts_hand_the_right_payload_to_a_compiled_plan():
    import lowbit_comm_b200 as lbc
    from lowbit_comm_b200.parallel.native_collectives import NativeCollectiveInput

    class Plan:
        def __init__(self):
            self.seen = []

        def run(self, payload):
            self.seen.append(payload)
            return ImmediateWork(payload)

    plan = Plan()
    a, b, c = object(), object(), object()
    assert lbc.all_reduce(a, compiled_plan=plan).wait() is a
    assert lbc.broadcast(a, src=1, compiled_plan=plan).wait() is a and lbc.reduce(a, dst=2, compiled_plan=plan).wait() is a
    lbc.all_gather(a, output_tensors=[b, c], compiled_plan=plan)
    lbc.gather(a, gather_list=[b], dst=1, compiled_plan=plan)
    lbc.reduce_scatter(a, input_tensors=[b, c], compiled_plan=plan)
    lbc.scatter(a, scatter_list=[b, c], src=0, compiled_plan=plan)
    lbc.all_to_all(output_tensors=[a], input_tensors=[b], compiled_plan=plan)
    lbc.barrier(compiled_plan=plan)
    lists = plan.seen[3:]
    assert all(isinstance(p, NativeCollectiveInput) for p in lists)
    assert (lists[0].tensor, lists[0].output_tensors, lists[0].input_tensors) == (a, (b, c), ())
    assert (lists[1].tensor, lists[1].output_tensors) == (a, (b,))
    assert (lists[2].tensor, lists[2].input_tensors) == (a, (b, c)) and lists[3].input_tensors == (b, c)
    assert (lists[4].tensor, lists[4].input_tensors, lists[4].output_tensors) == (None, (b,), (a,))
    assert lists[5] == NativeCollectiveInput()
    with pytest.raises(ValueError, match="at least one tensor"):
        lbc.all_to_all(output_tensors=[], input_tensors=[])
    assert lbc.native_collectives()[0] == "all_reduce" and len(lbc.native_collectives()) == 9


def test_plan_context_info_and_choice_helpers():
    from lowbit_comm_b200.core.backend import StrategyChoice
    from lowbit_comm_b200.core.info import ExecutionCounterSnapshot, ExecutionInfo
    from lowbit_comm_b200.core.plan import WorkspacePolicy

    plan = CommunicationPlan(collective="all_reduce", strategy="auto", backend="cuda", compression=CompressionConfig(),
                             fallback=("all_gather", "auto", "all_gather"))
    assert plan.key == ("all_reduce", "auto", "cuda", "full") and plan.is_compressed
    assert plan.candidates() == ("auto", "all_gather")
    assert not CommunicationPlan(collective="all_reduce", strategy="native_nccl", backend="cuda").is_compressed
    ctx = CompileContext(rank=5, world_size=8, device="cuda:1", shape=(4, 256), dtype="bf16", local_rank=1,
                         local_world_size=4, node_id=1, node_count=2)
    assert ctx.nbytes == 4 * 256 * 2 and ctx.has_node_layout
    assert not CompileContext(rank=0, world_size=8, device="cuda:0", shape=(1,), dtype="bf16").has_node_layout
    assert not CompileContext(rank=6, world_size=8, device="cuda:0", shape=(1,), dtype="bf16", local_rank=1,
                              local_world_size=4, node_id=1, node_count=2).has_node_layout
    policy = WorkspacePolicy(max_cached_bytes=100, max_entries=2)
    assert policy.admits(100, 2) and not policy.admits(101, 1) and not policy.admits(1, 3)
    assert WorkspacePolicy(cache=False).admits(0, 0) and not WorkspacePolicy(cache=False).admits(1, 1)

    info = ExecutionInfo(requested_strategy="auto", executed_strategy="all_gather", backend="cuda", fallback_used=True,
                         fallback_reason="ring missing", stage_names=("push", "reduce"), original_bytes=200,
                         compressed_bytes=104, compression_ratio=200 / 104, workspace_cache_hit=False,
                         async_capable=True, fast_path="fused")
    assert info.saved_bytes == 96 and info.with_details(note=1).details["note"] == 1 and not info.details
    text = info.summary()
    assert "auto -> all_gather (ring missing)" in text and "[push > reduce]" in text and "200 -> 104 bytes" in text
    assert ExecutionCounterSnapshot(5, 2, 1, 0, 0).in_flight == 2

    measured = StrategyChoice("reduce_scatter", "table hit", "p1", True, expected_speedup=1.25, evidence="profiles/x.md",
                              fallback=("native_nccl",))
    assert measured.speedup == 1.25
    assert measured.explain() == "reduce_scatter: table hit [p1]; 1.25x; evidence: profiles/x.md; then native_nccl"
    observed = StrategyChoice("compressed", "shard", "p1", False, observed_speedup=1.7, baseline="nccl full")
    assert "1.70x over nccl full" in observed.explain() and StrategyChoice("a", "b", "c", False).speedup is None
    for bad in (dict(expected_speedup=0.0), dict(observed_speedup=1.2), dict(benchmark_matched=True)):
        kwargs = {"benchmark_matched": False, **bad}
        matched = kwargs.pop("benchmark_matched")
        with pytest.raises(ValueError):
            StrategyChoice("a", "b", "c", matched, **kwargs)
    with pytest.raises(ValueError, match="positive integers"):
        BackendCapabilities(backend="x", available=True, bits=frozenset({0}))


def test_bound_all_reduce_settles_once_and_lets_go_of_a_closed_arena():
    """`Communicator.bind_all_reduce` (the compiled plan's hot path) resolves the workspace on the first call, reuses
    it while the arena it lives in is the communicator's live one, and resolves again after a close or when a
    tensor outgrows it; everything the fused kernels do not serve goes through `all_reduce`."""

    from lowbit_comm_b200.parallel.communicator import Communicator

    class Group:
        def __init__(self):
            self.checks = 0

        def check_status(self):
            self.checks += 1

    class Workspace:
        def __init__(self, group, max_numel):
            self.group, self.max_numel, self.calls = group, max_numel, []

        def all_reduce(self, tensor, out, *, op, stages):
            self.calls.append((tensor.numel(), op, stages))
            return tensor

    class Tensor:
        is_cuda = True

        def __init__(self, n):
            self._n = n

        def numel(self):
            return self._n

    comm = Communicator.__new__(Communicator)
    comm.transport, comm.peer_group, comm.stats, comm.closed = "auto", Group(), {"peer_ops": 0, "torch_ops": 0}, False
    made, slow = [], []
    comm.peer_usable = lambda tensor, config: True

    def workspace(tensor, config, dtype):
        made.append(Workspace(comm.peer_group, 1 << (tensor.numel() - 1).bit_length()))
        return made[-1]

    comm.workspace = workspace
    comm.all_reduce = lambda tensor, **kw: slow.append(kw["strategy"]) or tensor
    call = comm.bind_all_reduce(config=CompressionConfig(), op="mean", strategy="reduce_scatter", dtype="bf16")
    for n in (1000, 900, 1024):
        call(Tensor(n))
    assert len(made) == 1 and made[0].calls == [(1000, "mean", 2), (900, "mean", 2), (1024, "mean", 2)]
    assert comm.peer_group.checks == 2 and comm.stats["peer_ops"] == 3       # the first call checked inside workspace()
    call(Tensor(5000))                                                        # outgrown: resolved again
    assert len(made) == 2 and made[1].calls == [(5000, "mean", 2)]
    comm.peer_group = Group()                                                 # the arena was closed and made anew
    call(Tensor(10))
    assert len(made) == 3 and made[2].group is comm.peer_group and made[1].calls == [(5000, "mean", 2)]
    cpu = Tensor(10)
    cpu.is_cuda = False
    comm.peer_usable = lambda tensor, config: False
    call(cpu)
    assert slow == ["reduce_scatter"]
    with pytest.raises(UnsupportedCollective):
        comm.bind_all_reduce(config=CompressionConfig(), op="max")
    routed = comm.bind_all_reduce(config=CompressionConfig(), strategy="hierarchical")
    routed(Tensor(10))
    assert slow == ["reduce_scatter", "hierarchical"]
