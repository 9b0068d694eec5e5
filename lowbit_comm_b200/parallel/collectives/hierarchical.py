"""Hierarchical compressed all-reduce: reduce-scatter inside a local group, all-reduce of the shard across
groups, gather inside the group.

Routes, in order: the caller's `hierarchical_all_reduce` transport when one is injected, otherwise this
process' communicator (peer-memory kernels inside the group, compressed exchange across groups); then the
caller's `all_gather_fallback`, reached only when the first route declines.  The keyword names are the
reference's (ccdl_comm/collectives/hierarchical.py:10-55); `local_group_size` and `group` are additions.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ...config import CompressionConfig
from ._routes import check_reduction, first_that_serves, injected


def compressed_hierarchical_all_reduce(tensor: Any, *, config: CompressionConfig, op: str = "mean",
                                       async_op: bool = False, dtype: str = "auto",
                                       hierarchical_all_reduce: Callable[..., Any] | None = None,
                                       all_gather_fallback: Callable[..., Any] | None = None,
                                       extension_status: Any | None = None,
                                       local_group_size: int | None = None, group: Any | None = None) -> Any:
    check_reduction("hierarchical", op)
    request = {"config": config, "op": op, "async_op": async_op, "dtype": dtype}

    def native(t: Any) -> Any:
        from ..communicator import get_communicator

        return get_communicator(group).hierarchical_all_reduce(t, local_group_size=local_group_size, **request)

    request_with_status = {**request, "extension_status": extension_status}
    routes = [native if hierarchical_all_reduce is None else injected(hierarchical_all_reduce, request_with_status)]
    if all_gather_fallback is not None:
        routes.append(injected(all_gather_fallback, request_with_status))
    return first_that_serves(routes, tensor, what="hierarchical")
