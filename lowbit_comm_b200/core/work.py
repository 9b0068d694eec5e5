"""What every collective returns: something to `wait()` on, `query()`, and read compile-time facts from.

All three concrete kinds share one state machine, `_SettlesOnce`: the first `wait()` drives the work to its end
(`_drive`), the outcome -- a value or the exception that ended it -- is kept, and every later `wait()` replays
that outcome.  The end is reported to the shared `ExecutionCounters` exactly once, as completed or failed.

* `ImmediateWork`        the value already exists
* `CompletionWork`       transport handle, then a one-shot finishing callback, then a completion event; it also
                         keeps the buffers the transfer uses alive.  Python twin of the native `CompressedWork`
                         (ops/csrc/work.cpp)
* `BoundCollectiveWork`  somebody else's work-like object, reporting this framework's facts

Public names and semantics follow the reference (ccdl_comm/work.py:15-287).
"""

from __future__ import annotations

import threading
from collections.abc import Callable, Sequence
from typing import Any, Generic, TypeVar

from .info import ExecutionCounters, ExecutionInfo

T = TypeVar("T")

_PROBES = ("is_completed", "query")


def _method(obj: Any | None, name: str) -> Callable[[], Any] | None:
    found = getattr(obj, name, None)
    return found if callable(found) else None


def _block_on(obj: Any | None) -> None:
    """`obj.wait()` when there is such a thing; handles and events of unknown type are accepted."""

    wait = _method(obj, "wait")
    if wait is not None:
        wait()


def _poll(obj: Any | None) -> bool:
    """Non-blocking: has `obj` finished?  Nothing to wait for counts as finished; an object that cannot be
    asked counts as not finished."""

    if obj is None:
        return True
    probe = next(filter(None, (_method(obj, name) for name in _PROBES)), None)
    return bool(probe()) if probe is not None else False


def _future_of(obj: Any | None) -> Any | None:
    getter = _method(obj, "get_future")
    return None if getter is None else getter()


class CollectiveWork(Generic[T]):
    """The interface: `wait() -> result`, `query() -> bool`, optionally a future and compile-time facts."""

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


class _SettlesOnce(CollectiveWork[T]):
    """Shared wait/query bookkeeping.  Subclasses say how to reach the end (`_drive`) and how to peek
    (`_peek`); this class keeps the outcome, the counters and the lock."""

    def __init__(self, info: ExecutionInfo | None, counters: ExecutionCounters | None) -> None:
        self._info = info
        self._counters = counters
        self._settled = False
        self._value: Any = None
        self._error: BaseException | None = None
        self._reported = False
        self._lock = threading.Lock()
        self._driver: int | None = None      # thread that is inside _drive(), to catch a wait on itself

    # what subclasses provide
    def _drive(self) -> Any:
        raise NotImplementedError

    def _peek(self) -> bool:
        raise NotImplementedError

    @property
    def execution_info(self) -> ExecutionInfo | None:
        return self._info

    @property
    def execution_counters(self) -> ExecutionCounters | None:
        return self._counters

    def _note(self, event: str) -> None:
        if self._counters is not None:
            self._counters._bump(event)

    def _report_end(self) -> None:
        if self._settled and not self._reported and self._counters is not None:
            self._counters._bump("failed" if self._error is not None else "completed")
            self._reported = True

    def _settle(self, value: Any = None, error: BaseException | None = None) -> None:
        self._value, self._error, self._settled = value, error, True
        self._report_end()

    def wait(self) -> T:
        self._note("wait")
        if self._driver == threading.get_ident():
            raise RuntimeError("wait() was called by this work's own completion step; it would wait for itself")
        with self._lock:
            if not self._settled:
                self._driver = threading.get_ident()
                try:
                    outcome = self._drive()
                except BaseException as exc:      # kept: every later waiter sees the same failure
                    self._settle(error=exc)
                else:
                    self._settle(outcome)
                finally:
                    self._driver = None
        if self._error is not None:
            raise self._error
        return self._value

    def query(self) -> bool:
        self._note("query")
        return self._settled or self._peek()


class ImmediateWork(_SettlesOnce[T]):
    """A finished result behind the work interface.  Two of them are equal when their results are."""

    def __init__(self, result: T, execution_info: ExecutionInfo | None = None,
                 execution_counters: ExecutionCounters | None = None) -> None:
        super().__init__(execution_info, execution_counters)
        self._settle(result)

    @property
    def result(self) -> T:
        return self._value

    def _drive(self) -> T:
        return self._value

    def _peek(self) -> bool:
        return True

    def __eq__(self, other: object) -> bool:
        return isinstance(other, ImmediateWork) and self._value == other._value

    def __hash__(self) -> int:           # results may be unhashable tensors
        return id(self)

    def __repr__(self) -> str:
        return f"ImmediateWork(result={self._value!r})"


class CompletionWork(_SettlesOnce[T]):
    """Three things in order: the transport `handle`, the `complete` callback (runs once, its return value
    replaces `result`), the `completion` event.  `resources` are only held."""

    def __init__(self, result: T, *, handle: Any | None = None,
                 complete: Callable[[], T] | None = None, completion: Any | None = None,
                 resources: Sequence[Any] = (), execution_info: ExecutionInfo | None = None,
                 execution_counters: ExecutionCounters | None = None) -> None:
        super().__init__(execution_info, execution_counters)
        self._value = result
        self._handle, self._completion = handle, completion
        self._pending_callback = complete          # None once it has run (or when there is none)
        self._resources = tuple(resources)

    @property
    def resources(self) -> tuple[Any, ...]:
        return self._resources

    def _drive(self) -> T:
        _block_on(self._handle)
        finish, self._pending_callback = self._pending_callback, None
        if finish is not None:
            self._value = finish()
        _block_on(self._completion)
        return self._value

    def _peek(self) -> bool:
        return _poll(self._handle) and self._pending_callback is None and _poll(self._completion)

    def get_future(self) -> Any | None:
        return _future_of(self._handle)

    def _bind_execution(self, info: ExecutionInfo, counters: ExecutionCounters) -> None:
        if self._counters is not None and self._counters is not counters:
            raise ValueError("work already has different execution_counters")
        self._info, self._counters = info, counters
        self._report_end()                         # work that ended before it was bound still counts once


class BoundCollectiveWork(_SettlesOnce[T]):
    """A foreign work-like object (`wait` plus `query` or `is_completed`) that reports compiled facts."""

    def __init__(self, delegate: Any, execution_info: ExecutionInfo,
                 execution_counters: ExecutionCounters) -> None:
        super().__init__(execution_info, execution_counters)
        self._delegate = delegate

    @property
    def resources(self) -> tuple[Any, ...]:
        return tuple(getattr(self._delegate, "resources", ()))

    def _drive(self) -> T:
        return self._delegate.wait()

    def _peek(self) -> bool:
        return _poll(self._delegate)

    def get_future(self) -> Any | None:
        return _future_of(self._delegate)


def _is_work_like(obj: Any) -> bool:
    if isinstance(obj, CollectiveWork):
        return True
    return _method(obj, "wait") is not None and any(_method(obj, name) is not None for name in _PROBES)


def bind_execution_work(result: Any, execution_info: ExecutionInfo,
                        execution_counters: ExecutionCounters) -> CollectiveWork[Any]:
    """Whatever an executor's operation returned, as work that carries the executor's facts and counters:
    our own work kinds are re-labelled in place where that is safe, foreign ones are wrapped, plain values
    become `ImmediateWork`."""

    if isinstance(result, CompletionWork):
        result._bind_execution(execution_info, execution_counters)
        return result
    if isinstance(result, ImmediateWork):
        if result.execution_counters is execution_counters:     # already counted there: only the label changes
            result._info = execution_info
            return result
        result = result.result
    elif _is_work_like(result):
        return BoundCollectiveWork(result, execution_info, execution_counters)
    return ImmediateWork(result, execution_info, execution_counters)
