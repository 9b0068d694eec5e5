"""Work objects: Python `CompletionWork` and the native `CompressedWork` share one contract."""

import threading
import time

import pytest

from lowbit_comm_b200 import CompletionWork, ExecutionCounters, ExecutionInfo, ImmediateWork, bind_execution_work
from lowbit_comm_b200.core.work import BoundCollectiveWork
from lowbit_comm_b200.ops.loader import load_cuda_extension


def info():
    return ExecutionInfo(requested_strategy="a", executed_strategy="a", backend="cuda", fallback_used=False,
                         fallback_reason=None, stage_names=(), original_bytes=1, compressed_bytes=1,
                         compression_ratio=1.0, workspace_cache_hit=False, async_capable=True, fast_path="x")


class Handle:
    def __init__(self, fail=None, done=True):
        self.waits, self.fail, self.done = 0, fail, done

    def wait(self):
        self.waits += 1
        if self.fail:
            raise self.fail

    def is_completed(self):
        return self.done

    def get_future(self):
        return "future"


class Event:
    def __init__(self, ready=True):
        self.ready, self.waits = ready, 0

    def query(self):
        return self.ready

    def wait(self):
        self.waits += 1


def python_work(result, **kw):
    return CompletionWork(result, **kw)


def native_work(result, handle=None, complete=None, completion=None, resources=()):
    ext = load_cuda_extension()
    if not ext.available:
        pytest.skip(f"extension not built: {ext.reason}")
    return ext.module.CompressedWork(result, handle, completion, list(resources), complete)


FACTORIES = [("python", lambda r, **kw: python_work(r, **kw)),
             ("native", lambda r, **kw: native_work(r, kw.get("handle"), kw.get("complete"), kw.get("completion"),
                                                     kw.get("resources", ())))]


@pytest.mark.parametrize("name,make", FACTORIES)
def test_callback_runs_once_and_query_never_runs_it(name, make):
    calls = []
    handle, event = Handle(), Event()
    work = make("early", handle=handle, complete=lambda: calls.append(1) or "late", completion=event, resources=("buf",))
    assert not work.query() and calls == []          # callback pending: not done, and query did not run it
    assert work.wait() == "late" and work.wait() == "late"
    assert calls == [1] and handle.waits == 1 and event.waits == 1 and work.query()
    assert work.get_future() == "future"


@pytest.mark.parametrize("name,make", FACTORIES)
def test_first_error_is_cached_and_reraised(name, make):
    work = make("x", handle=Handle(fail=RuntimeError("link down")), complete=lambda: "never")
    for _ in range(3):
        with pytest.raises(RuntimeError, match="link down"):
            work.wait()
    assert work.query()
    boom = make("x", complete=lambda: (_ for _ in ()).throw(ValueError("bad callback")))
    with pytest.raises(ValueError, match="bad callback"):
        boom.wait()
    with pytest.raises(ValueError, match="bad callback"):
        boom.wait()


@pytest.mark.parametrize("name,make", FACTORIES)
def test_concurrent_waiters_see_one_completion(name, make):
    calls = []

    def slow():
        time.sleep(0.05)
        calls.append(1)
        return 42

    work = make(None, complete=slow)
    results = []
    threads = [threading.Thread(target=lambda: results.append(work.wait())) for _ in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(5)
    assert results == [42] * 8 and calls == [1]


def test_counters_and_binding():
    counters = ExecutionCounters()
    done = bind_execution_work("value", info(), counters)
    assert isinstance(done, ImmediateWork) and done.wait() == "value" and done.query()
    pending = bind_execution_work(CompletionWork("v", handle=Handle()), info(), counters)
    assert pending.execution_info.fast_path == "x" and pending.wait() == "v"
    failing = bind_execution_work(CompletionWork("v", handle=Handle(fail=OSError("x"))), info(), counters)
    with pytest.raises(OSError):
        failing.wait()
    foreign = bind_execution_work(Handle(), info(), counters)
    assert isinstance(foreign, BoundCollectiveWork) and foreign.query() and foreign.wait() is None
    snap = counters.snapshot()
    assert snap.completed_runs == 3 and snap.failed_runs == 1 and snap.wait_calls == 4 and snap.query_calls == 2
    with pytest.raises(ValueError):
        CompletionWork("v", execution_counters=ExecutionCounters())._bind_execution(info(), counters)


def test_execution_info_validation():
    base = dict(requested_strategy="a", executed_strategy="a", backend="cuda", fallback_used=False, fallback_reason=None,
                stage_names=(), original_bytes=1, compressed_bytes=1, compression_ratio=1.0, workspace_cache_hit=False,
                async_capable=True, fast_path="x")
    for bad in (dict(fallback_used=True), dict(fallback_reason="why"), dict(compression_ratio=0.0),
                dict(compression_ratio=float("inf")), dict(original_bytes=-1), dict(fast_path=""), dict(stage_names=("",))):
        with pytest.raises(ValueError):
            ExecutionInfo(**{**base, **bad})
    ok = ExecutionInfo(**{**base, "fallback_used": True, "fallback_reason": "no peer access", "details": {"k": 1}})
    with pytest.raises(TypeError):
        ok.details["k"] = 2


@pytest.mark.timeout(60)
@pytest.mark.parametrize("name,make", FACTORIES)
def test_a_completion_step_that_waits_on_its_own_work_is_an_error_not_a_deadlock(name, make):
    holder = {}
    work = make(None, complete=lambda: holder["work"].wait())
    holder["work"] = work
    with pytest.raises(RuntimeError, match="wait for itself"):
        work.wait()
    with pytest.raises(RuntimeError, match="wait for itself"):       # the failure is the work's outcome now
        work.wait()
    assert work.query()
