"""Backend conformance of the nine pass-through collectives, with a fake torch.distributed.

Mirrors the reference's conformance tier (tests/conformance/test_collective_protocol.py:16-60):
ordered protocol, sync/async work semantics, root and reduce-op binding, errors at compile time.
No torch, no process group: the fake records every call.
"""

import pytest

from lowbit_comm_b200.core.plan import CommunicationPlan, CompileContext
from lowbit_comm_b200.parallel.native_collectives import (NATIVE_COLLECTIVES, NativeCollectiveInput,
                                                          compile_native_collective)


class FakeHandle:
    def __init__(self, log, name):
        self.log, self.name, self.waited = log, name, 0

    def wait(self):
        self.waited += 1
        self.log.append(("wait", self.name))
        return True

    def is_completed(self):
        return self.waited > 0


class FakeTensor:
    def __init__(self, tag, shape=(4,)):
        self.tag, self.shape = tag, shape

    def new_empty(self, shape):
        return FakeTensor(f"{self.tag}.empty", tuple(shape))


class FakeDist:
    class ReduceOp:
        SUM, AVG, PRODUCT, MIN, MAX = "SUM", "AVG", "PRODUCT", "MIN", "MAX"

    def __init__(self):
        self.log = []

    def _call(self, name, async_op, **kw):
        self.log.append((name, kw))
        return FakeHandle(self.log, name) if async_op else None

    def all_reduce(self, t, op=None, async_op=False, **kw):
        return self._call("all_reduce", async_op, op=op, **kw)

    def all_gather(self, outs, t, async_op=False, **kw):
        return self._call("all_gather", async_op, outs=len(outs), **kw)

    def reduce_scatter(self, out, ins, op=None, async_op=False, **kw):
        return self._call("reduce_scatter", async_op, op=op, ins=len(ins), **kw)

    def all_to_all(self, outs, ins, async_op=False, **kw):
        return self._call("all_to_all", async_op, outs=len(outs), ins=len(ins), **kw)

    def broadcast(self, t, src=0, async_op=False, **kw):
        return self._call("broadcast", async_op, src=src, **kw)

    def reduce(self, t, dst=0, op=None, async_op=False, **kw):
        return self._call("reduce", async_op, dst=dst, op=op, **kw)

    def gather(self, t, gather_list=None, dst=0, async_op=False, **kw):
        return self._call("gather", async_op, dst=dst, outs=None if gather_list is None else len(gather_list), **kw)

    def scatter(self, out, scatter_list=None, src=0, async_op=False, **kw):
        return self._call("scatter", async_op, src=src, ins=None if scatter_list is None else len(scatter_list), **kw)

    def barrier(self, async_op=False, **kw):
        return self._call("barrier", async_op, **kw)

    def get_backend(self, group=None):
        return "gloo"


def _ctx(rank=1, world=4, **kw):
    return CompileContext(rank=rank, world_size=world, device="cuda:0", shape=(4,), dtype="bf16", **kw)


def _plan(collective, **kw):
    return CommunicationPlan(collective=collective, strategy="native_nccl", **kw)


def test_protocol_order_and_count():
    assert NATIVE_COLLECTIVES == ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "reduce",
                                  "gather", "scatter", "barrier")


@pytest.mark.parametrize("async_op", (True, False))
def test_every_collective_reaches_the_backend_once(async_op):
    world = 4
    t = FakeTensor("x")
    many = tuple(FakeTensor(f"p{i}") for i in range(world))
    inputs = {
        "all_reduce": t, "all_gather": t, "broadcast": t, "reduce": t, "barrier": None,
        "reduce_scatter": NativeCollectiveInput(tensor=t, input_tensors=many),
        "all_to_all": NativeCollectiveInput(input_tensors=many, output_tensors=many),
        "gather": NativeCollectiveInput(tensor=t, output_tensors=many),
        "scatter": NativeCollectiveInput(tensor=t, input_tensors=many),
    }
    for name in NATIVE_COLLECTIVES:
        dist = FakeDist()
        ctx = _ctx(rank=1, world=world)
        ex = compile_native_collective(_plan(name, async_op=async_op, root=1, reduce_op="sum"), ctx, dist=dist)
        work = ex.run(inputs[name])
        assert [c[0] for c in dist.log] == [name], name
        assert dist.log[0][1].get("async_op", async_op) == async_op or "async_op" not in dist.log[0][1]
        result = work.wait()
        assert work.query()
        if async_op:
            assert ("wait", name) in dist.log                       # the handle is waited exactly through the work
            work.wait()
            assert [c for c in dist.log if c == ("wait", name)] == [("wait", name)]   # and only once
        if name in ("all_reduce", "broadcast", "reduce"):
            assert result is t
        if name == "all_gather":
            assert len(result) == world
        assert ex.execution_info.fast_path == "cuda_native_nccl" and ex.execution_counters.snapshot().run_calls == 1


def test_root_and_reduce_op_are_bound_at_compile_time():
    dist = FakeDist()
    ex = compile_native_collective(_plan("reduce", root=2, reduce_op="max"), _ctx(), dist=dist)
    ex.run(FakeTensor("x")).wait()
    assert dist.log[0] == ("reduce", {"dst": 2, "op": "MAX"})
    dist = FakeDist()
    ex = compile_native_collective(_plan("broadcast", root=3), _ctx(), dist=dist)
    ex.run(FakeTensor("x")).wait()
    assert dist.log[0][1]["src"] == 3
    # non-root ranks of gather/scatter pass no lists
    dist = FakeDist()
    compile_native_collective(_plan("gather", root=0), _ctx(rank=1), dist=dist).run(FakeTensor("x")).wait()
    assert dist.log[0][1]["outs"] is None


def test_rejections_happen_at_compile_time():
    with pytest.raises(ValueError):
        compile_native_collective(_plan("all_reduce", root=9), _ctx(), dist=FakeDist())        # root outside the group
    with pytest.raises(ValueError):
        compile_native_collective(_plan("all_reduce", reduce_op="median"), _ctx(), dist=FakeDist())
    with pytest.raises(ValueError):
        compile_native_collective(_plan("ring_shuffle"), _ctx(), dist=FakeDist())
    with pytest.raises(ValueError):
        compile_native_collective(CommunicationPlan(collective="all_reduce", strategy="all_gather"), _ctx(),
                                  dist=FakeDist())
    from lowbit_comm_b200.exceptions import UnsupportedCollective

    with pytest.raises(UnsupportedCollective):
        compile_native_collective(_plan("all_reduce"), _ctx(), dist=FakeDist(), require_nccl=True)   # gloo group


def test_shape_errors_are_reported_at_run_time_and_counted():
    dist = FakeDist()
    ex = compile_native_collective(_plan("reduce_scatter", reduce_op="sum"), _ctx(), dist=dist)
    with pytest.raises(ValueError):
        ex.run(NativeCollectiveInput(tensor=FakeTensor("x"), input_tensors=(FakeTensor("a"),)))
    snap = ex.execution_counters.snapshot()
    assert snap.run_calls == 1 and snap.failed_runs == 1 and dist.log == []
