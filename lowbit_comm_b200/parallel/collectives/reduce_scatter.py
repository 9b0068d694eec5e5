"""`compressed_reduce_scatter` and the reduced-shard interface
(parity: ccdl_comm/collectives/reduce_scatter.py:19-115)."""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ...config import CompressionConfig
from ...core.shard import ReducedShard
from ...core.work import CollectiveWork, ImmediateWork
from ...exceptions import UnsupportedCollective


def _as_work(value: Any, async_op: bool) -> Any:
    is_work = callable(getattr(value, "wait", None)) and not hasattr(value, "shape") and not isinstance(value, ReducedShard)
    if async_op:
        return value if is_work else ImmediateWork(value)
    return value.wait() if is_work else value


def compressed_reduce_scatter(
    tensor: Any,
    *,
    config: CompressionConfig,
    op: str = "mean",
    async_op: bool = False,
    dtype: str = "auto",
    reduce_scatter: Callable[..., Any] | None = None,
    all_gather_fallback: Callable[..., Any] | None = None,
    extension_status: Any | None = None,
    group: Any | None = None,
) -> Any:
    """Full-layout result computed through a compressed reduce-scatter + gather.

    With an injected `reduce_scatter` transport that transport runs (or
    `all_gather_fallback` when it raises `UnsupportedCollective`); otherwise the
    group's communicator runs its two-stage path and returns the full tensor.
    """

    if op not in ("sum", "mean"):
        raise UnsupportedCollective(f"reduce_scatter:{op}", reason="only op='sum' and op='mean' are implemented")
    if reduce_scatter is not None:
        try:
            return _as_work(reduce_scatter(tensor, config=config, op=op, async_op=async_op, dtype=dtype,
                                           extension_status=extension_status), async_op)
        except UnsupportedCollective:
            if all_gather_fallback is None:
                raise
            return _as_work(all_gather_fallback(tensor, config=config, op=op, async_op=async_op, dtype=dtype,
                                                extension_status=extension_status), async_op)
    from ..communicator import get_communicator

    result = get_communicator(group).reduce_scatter_full(tensor, config=config, op=op, dtype=dtype)
    return _as_work(result, async_op)


def compressed_reduce_scatter_shard(
    tensor: Any,
    *,
    config: CompressionConfig,
    op: str = "mean",
    async_op: bool = False,
    dtype: str = "auto",
    reduce_scatter_shard: Callable[..., Any] | None = None,
    extension_status: Any | None = None,
    compiled_plan: Any | None = None,
    out: Any | None = None,
    group: Any | None = None,
) -> ReducedShard | CollectiveWork[ReducedShard]:
    """Reduce across ranks and keep only this rank's shard (for sharded optimizers).

    `out` may be a caller-owned flat tensor (or an output lease) that receives the
    shard; it is validated for shape, dtype, device, contiguity and aliasing.
    """

    if op not in ("sum", "mean"):
        raise UnsupportedCollective(f"reduce_scatter:{op}", reason="only op='sum' and op='mean' are implemented")
    if compiled_plan is not None:
        work = compiled_plan.run(tensor, out=out) if out is not None else compiled_plan.run(tensor)
        return _as_work(work, async_op)
    if reduce_scatter_shard is not None:
        kwargs = dict(config=config, op=op, async_op=async_op, dtype=dtype, extension_status=extension_status)
        if out is not None:
            kwargs["out"] = out
        return _as_work(reduce_scatter_shard(tensor, **kwargs), async_op)
    from ..communicator import get_communicator

    return get_communicator(group).reduce_scatter_shard(tensor, config=config, op=op, async_op=async_op,
                                                        dtype=dtype, out=out)
