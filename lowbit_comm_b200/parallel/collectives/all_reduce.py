"""`compressed_all_reduce` (parity: ccdl_comm/collectives/all_reduce.py:48-333)."""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ...config import CompressionConfig
from ...core.work import CollectiveWork, CompletionWork, ImmediateWork
from ...exceptions import UnsupportedCollective
from ...ops import codec
from ..payload import (CompressedAllGatherReduce, CompressedAllReduce, CompressedPayload, GatheredPayloads,
                       coerce_payload, payload_buffer)
from ..payload_packing import (DEFAULT_FUSED_PAYLOAD_MIN_NUMEL, make_fused_payload_all_gather,
                               make_payload_all_gather, should_fuse_payload)

_STRATEGIES = {"all_gather", "all_reduce", "topology", "reduce_scatter", "hierarchical", "auto", "native_nccl"}


def _finish(work_or_value: Any, async_op: bool) -> Any:
    is_work = callable(getattr(work_or_value, "wait", None)) and not hasattr(work_or_value, "shape")
    if async_op:
        return work_or_value if is_work else ImmediateWork(work_or_value)
    return work_or_value.wait() if is_work else work_or_value


def compressed_all_reduce(
    tensor: Any,
    *,
    config: CompressionConfig,
    op: str = "mean",
    strategy: str = "all_gather",
    async_op: bool = False,
    world_size: int | None = None,
    dtype: str = "auto",
    quantize: Callable[[Any, CompressionConfig], Any] | None = None,
    dequantize: Callable[[Any, tuple[int, ...], CompressionConfig, str], Any] | None = None,
    all_reduce: Callable[[CompressedPayload, str], CompressedPayload] | None = None,
    all_gather: Callable[[Any], GatheredPayloads] | None = None,
    topology_all_reduce: Callable[..., Any] | None = None,
    topology_method: str | None = None,
    fuse_payload: bool = False,
    fuse_payload_min_numel: int = DEFAULT_FUSED_PAYLOAD_MIN_NUMEL,
    extension_status: Any | None = None,
    completion_manager: Any | None = None,
    compiled_plan: Any | None = None,
    group: Any | None = None,
    out: Any | None = None,
) -> Any | CollectiveWork[Any]:
    """All-reduce `tensor` through the low-bit wire format.

    Without injected callables the call goes to the group's `Communicator`
    (fused peer-memory kernels on CUDA, torch.distributed + codec elsewhere) and
    the result is written in place unless `out` is given.  Injected `quantize`,
    `dequantize`, `all_gather`, `all_reduce` or `topology_all_reduce` callables
    select the generic composition the reference uses, which returns a new tensor.
    """

    if strategy not in _STRATEGIES:
        raise UnsupportedCollective(f"all_reduce:{strategy}", reason=f"supported strategies: {sorted(_STRATEGIES)}")
    if op not in ("sum", "mean"):
        raise UnsupportedCollective(f"all_reduce:{op}", reason="only op='sum' and op='mean' are implemented")
    if compiled_plan is not None:
        return _finish(compiled_plan.run(tensor), async_op)
    injected = any(v is not None for v in (quantize, dequantize, all_reduce, all_gather, topology_all_reduce))
    if not injected:
        from ..communicator import get_communicator

        comm = get_communicator(group, extension_status=extension_status) if extension_status is not None \
            else get_communicator(group)
        chosen = topology_method if (strategy == "topology" and topology_method) else strategy
        return comm.all_reduce(tensor, config=config, op=op, strategy=chosen, async_op=async_op, dtype=dtype, out=out)

    name = codec.resolve_dtype(dtype, tensor) if dtype == "auto" and hasattr(tensor, "dtype") and \
        not isinstance(getattr(tensor, "dtype"), str) else (dtype if dtype != "auto" else "fp32")
    shape = tuple(getattr(tensor, "shape", ()))

    def q(t: Any, cfg: CompressionConfig) -> CompressedPayload:
        raw = quantize(t, cfg) if quantize is not None else codec.quantize_tensor(t, cfg, extension_status=extension_status)
        return coerce_payload(raw, shape=tuple(getattr(t, "shape", shape)), dtype=name)

    def dq(payload: Any, shp: tuple[int, ...], cfg: CompressionConfig, nm: str) -> Any:
        if dequantize is not None:
            return dequantize(payload, shp, cfg, nm)
        return codec.dequantize_tensor(payload_buffer(payload), shp, cfg, dtype=nm, extension_status=extension_status)

    if strategy == "topology":
        if topology_all_reduce is None:
            raise UnsupportedCollective("all_reduce:topology", reason="no topology transport was injected")
        return _finish(topology_all_reduce(tensor, config=config, op=op, async_op=async_op, dtype=name,
                                           extension_status=extension_status), async_op)
    if strategy == "all_reduce":
        if all_reduce is None:
            raise UnsupportedCollective("all_reduce:all_reduce", reason="a payload all_reduce transport must be injected")
        pipeline = CompressedAllReduce(config=config, compress=q, all_reduce=all_reduce, decompress=dq)
        return _finish(pipeline.run(tensor, shape=shape, dtype=name, reduce=op), async_op)
    if all_gather is None:
        from ..torch_transport import make_torch_all_gather

        base = make_torch_all_gather(group=group)
        all_gather = make_fused_payload_all_gather(base) if should_fuse_payload(
            tensor, enabled=fuse_payload, min_numel=fuse_payload_min_numel) else make_payload_all_gather(base)
    pipeline = CompressedAllGatherReduce(config=config, compress=q, all_gather=all_gather, decompress=dq)
    if async_op:
        holder: dict[str, Any] = {}

        def complete() -> Any:
            holder["v"] = pipeline.run(tensor, shape=shape, dtype=name, reduce=op)
            return holder["v"]

        return CompletionWork(None, complete=complete)
    return pipeline.run(tensor, shape=shape, dtype=name, reduce=op)
