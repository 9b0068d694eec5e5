"""`compressed_hierarchical_all_reduce` (parity: ccdl_comm/collectives/hierarchical.py:10-55)."""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ...config import CompressionConfig
from ...exceptions import UnsupportedCollective


def compressed_hierarchical_all_reduce(
    tensor: Any,
    *,
    config: CompressionConfig,
    op: str = "mean",
    async_op: bool = False,
    dtype: str = "auto",
    hierarchical_all_reduce: Callable[..., Any] | None = None,
    all_gather_fallback: Callable[..., Any] | None = None,
    extension_status: Any | None = None,
    local_group_size: int | None = None,
    group: Any | None = None,
) -> Any:
    """Intra-group reduce-scatter, inter-group all-reduce of the shard, intra-group gather."""

    if op not in ("sum", "mean"):
        raise UnsupportedCollective(f"hierarchical:{op}", reason="only op='sum' and op='mean' are implemented")
    if hierarchical_all_reduce is not None:
        try:
            return hierarchical_all_reduce(tensor, config=config, op=op, async_op=async_op, dtype=dtype,
                                           extension_status=extension_status)
        except UnsupportedCollective:
            if all_gather_fallback is None:
                raise
            return all_gather_fallback(tensor, config=config, op=op, async_op=async_op, dtype=dtype,
                                       extension_status=extension_status)
    from ..communicator import get_communicator

    return get_communicator(group).hierarchical_all_reduce(tensor, config=config, op=op, async_op=async_op,
                                                           dtype=dtype, local_group_size=local_group_size)
