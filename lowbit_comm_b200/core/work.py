"""Asynchronous result objects returned by every collective.

Parity: ccdl_comm/work.py:15-287.  `CompletionWork` is the Python twin of the
native `CompressedWork` (ops/csrc/work.cpp): a transport handle, a one-shot
completion callback and a completion event, with the first error cached and
re-raised by every later `wait()`.
"""

from __future__ import annotations

import threading
from collections.abc import Callable, Sequence
from typing import Any, Generic, TypeVar

from .info import ExecutionCounters, ExecutionInfo

T = TypeVar("T")


def _ready(obj: Any | None) -> bool:
    """Non-blocking readiness probe for handles/events of unknown type."""

    if obj is None:
        return True
    for name in ("is_completed", "query"):
        probe = getattr(obj, name, None)
        if callable(probe):
            return bool(probe())
    return False


def _call_if_present(obj: Any | None, name: str) -> None:
    fn = getattr(obj, name, None)
    if callable(fn):
        fn()


class CollectiveWork(Generic[T]):
    """Protocol: `wait() -> result`, `query() -> bool`, optional future."""

    def wait(self) -> T:
        raise NotImplementedError

    def query(self) -> bool:
        raise NotImplementedError

    def get_future(self) -> Any | None:
        return None

    @property
    def execution_info(self) -> ExecutionInfo | None:
        return None

    @property
    def execution_counters(self) -> ExecutionCounters | None:
        return None


class ImmediateWork(CollectiveWork[T]):
    """An already-finished result behind the work interface."""

    __slots__ = ("result", "_info", "_counters")

    def __init__(self, result: T, execution_info: ExecutionInfo | None = None,
                 execution_counters: ExecutionCounters | None = None) -> None:
        self.result = result
        self._info = execution_info
        self._counters = execution_counters
        if execution_counters is not None:
            execution_counters._record_completed()

    @property
    def execution_info(self) -> ExecutionInfo | None:
        return self._info

    @property
    def execution_counters(self) -> ExecutionCounters | None:
        return self._counters

    def wait(self) -> T:
        if self._counters is not None:
            self._counters._record_wait()
        return self.result

    def query(self) -> bool:
        if self._counters is not None:
            self._counters._record_query()
        return True

    def __eq__(self, other: object) -> bool:
        return isinstance(other, ImmediateWork) and self.result == other.result

    def __hash__(self) -> int:  # results may be unhashable tensors
        return id(self)

    def __repr__(self) -> str:
        return f"ImmediateWork(result={self.result!r})"


class CompletionWork(CollectiveWork[T]):
    """Handle + deferred callback + completion event + retained buffers."""

    def __init__(self, result: T, *, handle: Any | None = None,
                 complete: Callable[[], T] | None = None, completion: Any | None = None,
                 resources: Sequence[Any] = (), execution_info: ExecutionInfo | None = None,
                 execution_counters: ExecutionCounters | None = None) -> None:
        self._result = result
        self._handle = handle
        self._complete = complete
        self._completion = completion
        self._resources = tuple(resources)
        self._callback_done = complete is None
        self._finished = False
        self._error: BaseException | None = None
        self._info = execution_info
        self._counters = execution_counters
        self._terminal_counted = False
        self._lock = threading.Lock()

    @property
    def resources(self) -> tuple[Any, ...]:
        return self._resources

    @property
    def execution_info(self) -> ExecutionInfo | None:
        return self._info

    @property
    def execution_counters(self) -> ExecutionCounters | None:
        return self._counters

    def _bind_execution(self, info: ExecutionInfo, counters: ExecutionCounters) -> None:
        if self._counters is not None and self._counters is not counters:
            raise ValueError("work already has different execution_counters")
        self._info, self._counters = info, counters
        if self._finished:
            self._count_terminal()

    def wait(self) -> T:
        if self._counters is not None:
            self._counters._record_wait()
        with self._lock:
            if not self._finished:
                try:
                    _call_if_present(self._handle, "wait")
                    if not self._callback_done:
                        self._result = self._complete()  # type: ignore[misc]
                        self._callback_done = True
                    _call_if_present(self._completion, "wait")
                except BaseException as exc:  # cached for every later waiter
                    self._error = exc
                finally:
                    self._finished = True
                    self._count_terminal()
        if self._error is not None:
            raise self._error
        return self._result

    def query(self) -> bool:
        if self._counters is not None:
            self._counters._record_query()
        if self._finished:
            return True
        return _ready(self._handle) and self._callback_done and _ready(self._completion)

    def get_future(self) -> Any | None:
        getter = getattr(self._handle, "get_future", None)
        return getter() if callable(getter) else None

    def _count_terminal(self) -> None:
        if self._terminal_counted or self._counters is None:
            return
        (self._counters._record_failed if self._error is not None else self._counters._record_completed)()
        self._terminal_counted = True


class BoundCollectiveWork(CollectiveWork[T]):
    """Wraps a foreign work-like object so it reports compiled metadata."""

    def __init__(self, delegate: Any, execution_info: ExecutionInfo,
                 execution_counters: ExecutionCounters) -> None:
        self._delegate = delegate
        self._info = execution_info
        self._counters = execution_counters
        self._finished = False
        self._result: Any = None
        self._error: BaseException | None = None

    @property
    def execution_info(self) -> ExecutionInfo:
        return self._info

    @property
    def execution_counters(self) -> ExecutionCounters:
        return self._counters

    @property
    def resources(self) -> tuple[Any, ...]:
        return tuple(getattr(self._delegate, "resources", ()))

    def wait(self) -> T:
        self._counters._record_wait()
        if not self._finished:
            try:
                self._result = self._delegate.wait()
                self._counters._record_completed()
            except BaseException as exc:
                self._error = exc
                self._counters._record_failed()
            finally:
                self._finished = True
        if self._error is not None:
            raise self._error
        return self._result

    def query(self) -> bool:
        self._counters._record_query()
        return True if self._finished else _ready(self._delegate)

    def get_future(self) -> Any | None:
        getter = getattr(self._delegate, "get_future", None)
        return getter() if callable(getter) else None


def bind_execution_work(result: Any, execution_info: ExecutionInfo,
                        execution_counters: ExecutionCounters) -> CollectiveWork[Any]:
    """Attach an executor's metadata/counters to whatever its operation returned."""

    if isinstance(result, ImmediateWork):
        if result.execution_counters is execution_counters:
            result._info = execution_info
            return result
        return ImmediateWork(result.result, execution_info, execution_counters)
    if isinstance(result, CompletionWork):
        result._bind_execution(execution_info, execution_counters)
        return result
    looks_like_work = callable(getattr(result, "wait", None)) and (
        callable(getattr(result, "query", None)) or callable(getattr(result, "is_completed", None)))
    if isinstance(result, CollectiveWork) or looks_like_work:
        return BoundCollectiveWork(result, execution_info, execution_counters)
    return ImmediateWork(result, execution_info, execution_counters)
