"""Three-stage hierarchical compilation for 8 ranks as 2 nodes x 4, without hardware: every rank's view,
with fake groups and recorded operations (the reference's tier: tests/cuda/test_hierarchical_stage_executor.py)."""

import pytest

from lowbit_comm_b200 import CommunicationPlan, CommunicationStage, CompileContext, CompressionConfig
from lowbit_comm_b200.core.hierarchy import (CompiledStage, HierarchicalExecutor, StageExecution,
                                             all_hierarchy_groups, canonical_hierarchical_stages,
                                             compile_hierarchical_stages, rank_topology)
from lowbit_comm_b200.exceptions import UnsupportedCollective

CFG = CompressionConfig()


class FakeGroup:
    def __init__(self, ranks):
        self.ranks = tuple(ranks)


class FakeCompletion:
    def __init__(self, log, name, ready=True):
        self.log, self.name, self.ready = log, name, ready

    def wait_stream(self, stream):
        self.log.append(("wait_stream", self.name, stream))

    def wait(self):
        self.log.append(("host_wait", self.name))

    def query(self):
        return self.ready


def _plan(stages=None):
    return CommunicationPlan(collective="all_reduce", strategy="hierarchical", compression=CFG,
                             stages=stages if stages is not None else canonical_hierarchical_stages(CFG))


def _ctx(rank, n=1003):
    return CompileContext(rank=rank, world_size=8, device="cuda:0", shape=(n,), dtype="bf16", local_rank=rank % 4,
                          local_world_size=4, node_id=rank // 4, node_count=2)


@pytest.mark.parametrize("rank", range(8))
def test_every_rank_sees_local_inter_local(rank):
    made, bound, log = [], [], []

    def group_factory(ranks):
        made.append(tuple(ranks))
        return FakeGroup(ranks)

    def operation_factory(stage, stage_ctx):
        bound.append((stage.name, stage_ctx.rank, stage_ctx.world_size, stage_ctx.shape, stage_ctx.process_group.ranks))

        def operation(value):
            log.append(("run", stage.name, value))
            return f"{stage.name}({value})"

        return operation

    executor = compile_hierarchical_stages(
        _plan(), _ctx(rank), operation_factory=operation_factory, group_members=lambda g: g.ranks,
        group_factory=group_factory, stream_factory=lambda stage, c: f"stream:{stage.name}",
        completion_factory=lambda stream: FakeCompletion(log, stream))
    # all ranks create all six groups in the same order: group creation is collective
    assert made == [(0, 1, 2, 3), (4, 5, 6, 7), (0, 4), (1, 5), (2, 6), (3, 7)]
    node, lane = rank // 4, rank % 4
    local = tuple(range(4 * node, 4 * node + 4))
    assert [(s.name, s.participants) for s in executor.stages] == [
        ("local_reduce_scatter", local), ("inter_all_reduce", (lane, 4 + lane)), ("local_all_gather", local)]
    assert [(s.input_layout, s.output_layout) for s in executor.stages] == [("full", "shard"), ("shard", "shard"),
                                                                            ("shard", "full")]
    # group-local rank and world 4 -> 2 -> 4; the shard is ceil(1003 / 4) elements between the local stages
    assert bound == [("local_reduce_scatter", lane, 4, (1003,), local),
                     ("inter_all_reduce", node, 2, (251,), (lane, 4 + lane)),
                     ("local_all_gather", lane, 4, (251,), local)]
    assert executor.stages[0].process_group is executor.stages[2].process_group
    assert (executor.input_layout, executor.output_layout) == ("full", "full")

    work = executor.run("grad")
    assert work.wait() == "local_all_gather(inter_all_reduce(local_reduce_scatter(grad)))"
    # no host wait between stages: each later stage's stream waits on the completion of the one before; the
    # only host wait is the caller's own wait() on the last stage
    assert [e for e in log if e[0] != "run"] == [("wait_stream", "stream:local_reduce_scatter", "stream:inter_all_reduce"),
                                                 ("wait_stream", "stream:inter_all_reduce", "stream:local_all_gather"),
                                                 ("host_wait", "stream:local_all_gather")]


def test_groups_given_by_the_plan_or_the_context_are_used_and_verified():
    local, inter = FakeGroup((4, 5, 6, 7)), FakeGroup((2, 6))
    stages = list(canonical_hierarchical_stages(CFG, inter_strategy="reduce_scatter", gather_strategy="compressed"))
    stages[1] = CommunicationStage("inter_all_reduce", "all_reduce", "reduce_scatter", compression=CFG,
                                   process_group=inter, output_layout="shard", async_op=False)
    ctx = CompileContext(rank=6, world_size=8, device="cuda:0", shape=(64,), dtype="bf16", local_rank=2,
                         local_world_size=4, node_id=1, node_count=2,
                         process_groups={"local_reduce_scatter": local, "local_all_gather": local})
    ex = compile_hierarchical_stages(_plan(tuple(stages)), ctx, operation_factory=lambda s, c: (lambda v: v),
                                     group_members=lambda g: g.ranks)
    assert [s.process_group for s in ex.stages] == [local, inter, local]
    wrong = CompileContext(rank=6, world_size=8, device="cuda:0", shape=(64,), dtype="bf16", local_rank=2,
                           local_world_size=4, node_id=1, node_count=2,
                           process_groups={"local_reduce_scatter": FakeGroup((0, 1, 2, 3)), "local_all_gather": local})
    with pytest.raises(ValueError, match="do not match expected ranks"):
        compile_hierarchical_stages(_plan(tuple(stages)), wrong, operation_factory=lambda s, c: (lambda v: v),
                                    group_members=lambda g: g.ranks)
    with pytest.raises(ValueError, match="process group or group factory"):
        compile_hierarchical_stages(_plan(), _ctx(0), operation_factory=lambda s, c: (lambda v: v),
                                    group_members=lambda g: g.ranks)


def test_rejections():
    ok = dict(operation_factory=lambda s, c: (lambda v: v), group_members=lambda g: g.ranks, group_factory=FakeGroup)
    with pytest.raises(ValueError, match="strategy='hierarchical'"):
        compile_hierarchical_stages(CommunicationPlan(collective="all_reduce", strategy="all_gather", compression=CFG),
                                    _ctx(0), **ok)
    with pytest.raises(ValueError, match="three-stage chain"):
        compile_hierarchical_stages(_plan(canonical_hierarchical_stages(CFG)[:2]), _ctx(0), **ok)
    swapped = canonical_hierarchical_stages(CFG)
    with pytest.raises(ValueError, match="three-stage chain"):
        compile_hierarchical_stages(_plan((swapped[1], swapped[0], swapped[2])), _ctx(0), **ok)
    flat = CompileContext(rank=0, world_size=8, device="cuda:0", shape=(8,), dtype="bf16")
    with pytest.raises(ValueError, match="local rank and world size"):
        compile_hierarchical_stages(_plan(), flat, **ok)
    odd = CompileContext(rank=5, world_size=8, device="cuda:0", shape=(8,), dtype="bf16", local_rank=2,
                         local_world_size=4, node_id=1, node_count=2)
    with pytest.raises(ValueError, match="inconsistent"):
        rank_topology(odd)
    with pytest.raises(TypeError):
        compile_hierarchical_stages(_plan(), _ctx(0), operation_factory=None)
    assert all_hierarchy_groups(_ctx(3))[2:4] == ((0, 4), (1, 5))


def test_executor_chain_checks_quarantine_and_explicit_stage_results():
    log = []
    a = CompiledStage("a", "full", "shard", (0, 1), object(), lambda v: StageExecution(v + 1, FakeCompletion(log, "a"), (v,)))
    b = CompiledStage("b", "shard", "full", (0, 1), object(), lambda v: v * 10)
    assert HierarchicalExecutor([a, b]).run(1).wait() == 20
    assert ("host_wait", "a") in log          # stage b has no stream: it falls back to a host wait on the dependency
    with pytest.raises(ValueError, match="layout mismatch"):
        HierarchicalExecutor([b, b])
    with pytest.raises(ValueError):
        HierarchicalExecutor([])
    with pytest.raises(UnsupportedCollective):
        # a chain whose first stage starts from the wrong layout for its collective
        bad = (CommunicationStage("x", "reduce_scatter", "compressed", compression=CFG, output_layout="shard", async_op=False),
               CommunicationStage("y", "all_reduce", "topology", compression=CFG, output_layout="shard", async_op=False),
               CommunicationStage("z", "all_gather", "native_nccl", output_layout="full", async_op=False))
        plan = CommunicationPlan(collective="all_reduce", strategy="hierarchical", compression=CFG, stages=bad)
        import lowbit_comm_b200.core.hierarchy as h

        saved = dict(h._TRANSITIONS)
        try:
            h._TRANSITIONS.pop(("all_reduce", "shard", "shard"))
            compile_hierarchical_stages(plan, _ctx(0), operation_factory=lambda s, c: (lambda v: v),
                                        group_members=lambda g: g.ranks, group_factory=FakeGroup)
        finally:
            h._TRANSITIONS.update(saved)

    pending = FakeCompletion(log, "fence", ready=False)

    def boom(v):
        raise RuntimeError("stage failed")

    failing = HierarchicalExecutor([CompiledStage("a", "full", "shard", (0, 1), object(), lambda v: v),
                                    CompiledStage("b", "shard", "full", (0, 1), object(), boom,
                                                  completion_factory=lambda stream: pending)])
    with pytest.raises(RuntimeError):
        failing.run("x")
    assert failing.pending_failure_count == 1 and failing.reap_pending_failures() == 0   # device work not finished
    pending.ready = True
    assert failing.reap_pending_failures() == 1 and failing.pending_failure_count == 0
