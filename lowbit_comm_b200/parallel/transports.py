"""Transport factories with the reference's names and calling convention.

The reference builds its reduce-scatter, topology (ring / tree / p2p / overlap-*) and hierarchical paths as
factories that return `transport(tensor, *, config, op, async_op, dtype, extension_status[, out])`, and
injects them into the public collectives and into `create_ddp_comm_hook`
(ccdl_comm/communication/reduce_scatter_transport.py:18-130, topology_transport.py:14-200,
hierarchical_transport.py:106-200).  Code written against those factories keeps working here: the
factories below return callables of the same shape.  What runs behind them is different: every one maps
onto the `Communicator` of its process group, i.e. onto the fused push / reduce kernels over NVLink when
the tensors are on CUDA and onto the same staging through torch.distributed otherwise.  On an NVSwitch
node every peer is one hop away, so the ring, tree and pairwise schedules of the reference collapse into
the one-stage and two-stage direct exchanges; the method names are accepted and select between those two.
The ring and the tree also exist as real hop-by-hop executors (`parallel/schedule_executors.py`), for groups
that span nodes or have no peer access; `make_native_topology_all_reduce(hop_by_hop=True)` selects them.
Arguments that only made sense for the reference's host-driven schedules (workspace allocators, chunk
plans, fused-kernel switches, future factories) are accepted and ignored.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ..config import CompressionConfig
from ..exceptions import UnsupportedCollective

# the reference's method names -> the exchange that serves them here
ONE_STAGE_METHODS = frozenset({"all_gather", "gather", "overlap-gather"})
TWO_STAGE_METHODS = frozenset({"ring", "tree", "p2p", "butterfly", "overlap-p2p", "overlap-tree", "overlap-scale",
                               "topology", "reduce_scatter", "compressed"})


def _communicator(group: Any):
    from .communicator import get_communicator

    return get_communicator(group)


def _strategy_for(method: str | None) -> str:
    if method is None:
        return "auto"
    if method in ONE_STAGE_METHODS:
        return "all_gather"
    if method in TWO_STAGE_METHODS:
        return "reduce_scatter"
    raise UnsupportedCollective(f"topology:{method}", reason="unknown topology method")


def _check_op(op: str, what: str) -> None:
    if op not in ("sum", "mean"):
        raise UnsupportedCollective(f"{what}:{op}", reason="only op='sum' and op='mean' are implemented")


def make_torch_compressed_reduce_scatter_shard(*, group: Any | None = None, **_ignored: Any) -> Callable[..., Any]:
    """transport(...) -> `ReducedShard` (or a work object when `async_op`); honours a caller-owned `out`."""

    def transport(tensor: Any, *, config: CompressionConfig, op: str, async_op: bool, dtype: str,
                  extension_status: Any | None = None, out: Any | None = None) -> Any:
        _check_op(op, "reduce_scatter")
        return _communicator(group).reduce_scatter_shard(tensor, config=config, op=op, async_op=async_op,
                                                         dtype=dtype, out=out)

    return transport


def make_torch_compressed_reduce_scatter_all_gather(*, group: Any | None = None, **_ignored: Any) -> Callable[..., Any]:
    """transport(...) -> the full reduced tensor: compressed reduce-scatter, then the shards are gathered back
    (here also compressed: the two-stage all-reduce)."""

    def transport(tensor: Any, *, config: CompressionConfig, op: str, async_op: bool, dtype: str,
                  extension_status: Any | None = None) -> Any:
        _check_op(op, "reduce_scatter")
        return _communicator(group).all_reduce(tensor.clone(), config=config, op=op, strategy="reduce_scatter",
                                               async_op=async_op, dtype=dtype)

    return transport


def make_native_topology_all_reduce(*, method: str | None = None, group: Any | None = None,
                                    hop_by_hop: bool = False, **_ignored: Any) -> Callable[..., Any]:
    """transport(...) -> the full reduced tensor; `method` is one of the reference's topology names.
    `hop_by_hop=True` (an addition) runs the method as named through torch.distributed instead of the direct
    exchange: "ring", "tree", "p2p", "butterfly" as schedules of point-to-point operations (the choice for groups
    that span nodes or have no peer access), "overlap-scale" as a library int8 all-reduce under a shared scale."""

    strategy = _strategy_for(method)
    if hop_by_hop:
        from .schedule_executors import make_schedule_all_reduce

        if method == "overlap-scale":
            from .shared_scale import make_shared_scale_all_reduce

            return make_shared_scale_all_reduce(group=group)
        hops = {None: "ring", "overlap-p2p": "p2p", "overlap-tree": "tree"}.get(method, method)
        return make_schedule_all_reduce(method=hops, group=group)

    # The reference's overlap-* methods start the exchange and leave its last step to `wait()`
    # (ccdl_comm/communication/topology_transport.py:53-107, 524-748).  Here an overlap-* call is always issued
    # on the communicator's side stream, whatever `async_op` says, and joined when the work is waited for: a
    # synchronous caller gets the result after that join, an asynchronous one gets the work object.
    overlapped = bool(method) and str(method).startswith("overlap-")

    def transport(tensor: Any, *, config: CompressionConfig, op: str, async_op: bool, dtype: str,
                  extension_status: Any | None = None) -> Any:
        _check_op(op, "topology_all_reduce")
        work = _communicator(group).all_reduce(tensor.clone(), config=config, op=op, strategy=strategy,
                                               async_op=async_op or overlapped, dtype=dtype)
        if overlapped and not async_op and hasattr(work, "wait"):
            return work.wait()
        return work

    transport.overlapped = overlapped
    return transport


def make_native_topology_reduce_scatter_shard(*, method: str | None = None, group: Any | None = None,
                                              hop_by_hop: bool = False, **_ignored: Any) -> Callable[..., Any]:
    """transport(...) -> `ReducedShard`.  Unlike the reference's ring, sizes need not divide by the world size.
    `hop_by_hop=True` runs the "ring" or "p2p" reduce-scatter over point-to-point operations."""

    _strategy_for(method)   # validates the name; without hop_by_hop every method is the same direct scatter
    if hop_by_hop:
        from .schedule_executors import make_schedule_reduce_scatter_shard

        return make_schedule_reduce_scatter_shard(method={None: "p2p", "overlap-p2p": "p2p"}.get(method, method),
                                                  group=group)

    def transport(tensor: Any, *, config: CompressionConfig, op: str, async_op: bool, dtype: str,
                  extension_status: Any | None = None, out: Any | None = None) -> Any:
        _check_op(op, "topology_reduce_scatter")
        return _communicator(group).reduce_scatter_shard(tensor, config=config, op=op, async_op=async_op,
                                                         dtype=dtype, out=out)

    return transport


def make_torch_hierarchical_all_reduce(*, local_group_size: int = 2, group: Any | None = None,
                                       **_ignored: Any) -> Callable[..., Any]:
    """transport(...) -> the full reduced tensor through the three-stage hierarchy (local reduce-scatter,
    inter-group all-reduce of the shard, local all-gather).  Asynchronous use is supported, unlike the
    reference's prototype."""

    if isinstance(local_group_size, bool) or not isinstance(local_group_size, int) or local_group_size <= 0:
        raise ValueError("local_group_size must be a positive integer")

    def transport(tensor: Any, *, config: CompressionConfig, op: str, async_op: bool, dtype: str,
                  extension_status: Any | None = None) -> Any:
        _check_op(op, "hierarchical")
        return _communicator(group).hierarchical_all_reduce(tensor, config=config, op=op, async_op=async_op,
                                                            dtype=dtype, local_group_size=local_group_size)

    return transport


make_legacy_topology_all_reduce = make_native_topology_all_reduce   # the pre-refactor name, same behaviour here
