"""How the public collective entry points pick an implementation.

Each entry point builds a short list of routes -- callables of the tensor -- and `first_that_serves` runs
them in order.  A route declines by raising `UnsupportedCollective`; the next route is then tried, and the
last refusal is what the caller sees when none serves.  Injected transports (the `all_gather=`,
`reduce_scatter=`, `hierarchical_all_reduce=` ... keyword arguments) receive the request as keyword
arguments, which is the calling convention the reference's transports are written against
(ccdl_comm/collectives/all_gather.py:27-93).
"""

from __future__ import annotations

from collections.abc import Callable, Iterable
from typing import Any

from ...core.shard import ReducedShard
from ...core.work import ImmediateWork
from ...exceptions import UnsupportedCollective

Route = Callable[[Any], Any]
REDUCTIONS = ("sum", "mean")


def check_reduction(collective: str, op: str) -> None:
    if op not in REDUCTIONS:
        raise UnsupportedCollective(f"{collective}:{op}", reason="only op='sum' and op='mean' are implemented")


def injected(transport: Callable[..., Any], request: dict[str, Any], **extra: Any) -> Route:
    """Route through a caller-provided transport: `transport(tensor, **request, **extra)`; entries of
    `extra` that are None are not passed."""

    passed = {**request, **{name: value for name, value in extra.items() if value is not None}}
    return lambda tensor: transport(tensor, **passed)


def first_that_serves(routes: Iterable[Route], tensor: Any, *, what: str) -> Any:
    refusal: UnsupportedCollective | None = None
    for route in routes:
        try:
            return route(tensor)
        except UnsupportedCollective as declined:
            refusal = declined
    raise refusal or UnsupportedCollective(f"{what}:transport", reason=f"no {what} route is configured")


def is_work(value: Any) -> bool:
    """Something to wait on, as opposed to a tensor or a reduced shard (tensors have `wait` too on some
    builds, hence the `shape` test)."""

    return callable(getattr(value, "wait", None)) and not hasattr(value, "shape") \
        and not isinstance(value, ReducedShard)


def as_requested(value: Any, async_op: bool) -> Any:
    """Work for an asynchronous request, a finished value for a synchronous one, whichever the route gave."""

    if async_op:
        return value if is_work(value) else ImmediateWork(value)
    return value.wait() if is_work(value) else value
