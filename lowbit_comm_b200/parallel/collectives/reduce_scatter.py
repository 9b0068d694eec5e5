"""Compressed reduce-scatter, with the result either re-assembled on every rank (`compressed_reduce_scatter`)
or left as this rank's shard (`compressed_reduce_scatter_shard`, for sharded optimizers).

Routes of the full-layout call: an injected `reduce_scatter` transport, or else the communicator's two-stage
peer-memory path; then `all_gather_fallback` when the first declines.  Routes of the shard call: a compiled
plan when the caller holds one, else an injected `reduce_scatter_shard` transport, else the communicator.
`out` may be a caller-owned flat tensor (or an output lease) that receives the shard; whoever serves the call
validates its shape, dtype, device, contiguity and aliasing.  Keyword names are the reference's
(ccdl_comm/collectives/reduce_scatter.py:19-115); `group` is an addition.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ...config import CompressionConfig
from ...core.shard import ReducedShard
from ...core.work import CollectiveWork
from ._routes import as_requested, check_reduction, first_that_serves, injected


def _communicator(group: Any | None):
    from ..communicator import get_communicator

    return get_communicator(group)


def compressed_reduce_scatter(tensor: Any, *, config: CompressionConfig, op: str = "mean", async_op: bool = False,
                              dtype: str = "auto", reduce_scatter: Callable[..., Any] | None = None,
                              all_gather_fallback: Callable[..., Any] | None = None,
                              extension_status: Any | None = None, group: Any | None = None) -> Any:
    check_reduction("reduce_scatter", op)
    request = {"config": config, "op": op, "async_op": async_op, "dtype": dtype,
               "extension_status": extension_status}
    if reduce_scatter is None:
        routes = [lambda t: _communicator(group).reduce_scatter_full(t, config=config, op=op, dtype=dtype)]
    else:
        routes = [injected(reduce_scatter, request)]
    if all_gather_fallback is not None:
        routes.append(injected(all_gather_fallback, request))
    return as_requested(first_that_serves(routes, tensor, what="reduce_scatter"), async_op)


def compressed_reduce_scatter_shard(tensor: Any, *, config: CompressionConfig, op: str = "mean",
                                    async_op: bool = False, dtype: str = "auto",
                                    reduce_scatter_shard: Callable[..., Any] | None = None,
                                    extension_status: Any | None = None, compiled_plan: Any | None = None,
                                    out: Any | None = None,
                                    group: Any | None = None) -> ReducedShard | CollectiveWork[ReducedShard]:
    check_reduction("reduce_scatter", op)
    into = {} if out is None else {"out": out}
    if compiled_plan is not None:
        route = lambda t: compiled_plan.run(t, **into)                                     # noqa: E731
    elif reduce_scatter_shard is not None:
        route = injected(reduce_scatter_shard, {"config": config, "op": op, "async_op": async_op, "dtype": dtype,
                                                "extension_status": extension_status}, **into)
    else:
        route = lambda t: _communicator(group).reduce_scatter_shard(                       # noqa: E731
            t, config=config, op=op, async_op=async_op, dtype=dtype, out=out)
    return as_requested(route(tensor), async_op)
