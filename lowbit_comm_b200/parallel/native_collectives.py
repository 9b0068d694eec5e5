"""Uncompressed pass-through collectives behind the Work/ExecutionInfo protocol.

Parity: ccdl_comm/cuda/native_collectives.py:21-338 (nine collectives, reduce
ops sum/mean(avg)/product/min/max, `NativeCollectiveInput`, compile-time
validation) and ccdl_comm/collectives/api.py:14-337 (public shortcuts).  NCCL
(or gloo on CPU) does the transfer; these exist so that every collective a
trainer needs flows through one API and reports the same metadata.
"""

from __future__ import annotations

from dataclasses import dataclass
from importlib import import_module
from typing import Any, Callable

from ..core.info import ExecutionCounters, ExecutionInfo
from ..core.plan import CommunicationPlan, CompileContext
from ..core.work import CompletionWork, bind_execution_work

_REDUCE_ALIASES = {"sum": "SUM", "mean": "AVG", "avg": "AVG", "product": "PRODUCT", "prod": "PRODUCT",
                   "min": "MIN", "max": "MAX"}


@dataclass(frozen=True)
class NativeCollectiveInput:
    tensor: object | None = None
    input_tensors: tuple[object, ...] = ()
    output_tensors: tuple[object, ...] = ()

    def __post_init__(self) -> None:
        object.__setattr__(self, "input_tensors", tuple(self.input_tensors))
        object.__setattr__(self, "output_tensors", tuple(self.output_tensors))


def _reduce_op(dist: Any, name: str, backend_is_gloo: bool = False):
    key = _REDUCE_ALIASES.get(name.strip().lower())
    if key is None:
        raise ValueError(f"unsupported reduce op {name!r}; expected one of {sorted(set(_REDUCE_ALIASES))}")
    return getattr(dist.ReduceOp, key)


def _kw(ctx: CompileContext, plan: CommunicationPlan) -> dict:
    kw: dict[str, Any] = {"async_op": plan.async_op}
    if ctx.process_group is not None:
        kw["group"] = ctx.process_group
    return kw


def _need_tensor(inv: NativeCollectiveInput, what: str):
    if inv.tensor is None:
        raise ValueError(f"{what} needs a tensor")
    return inv.tensor


def _b_all_reduce(plan, ctx, dist):
    op = _reduce_op(dist, plan.reduce_op)

    def run(inv):
        t = _need_tensor(inv, "all_reduce")
        return t, dist.all_reduce(t, op=op, **_kw(ctx, plan))

    return run


def _b_all_gather(plan, ctx, dist):
    def run(inv):
        t = _need_tensor(inv, "all_gather")
        outs = list(inv.output_tensors) or [t.new_empty(t.shape) for _ in range(ctx.world_size)]
        if len(outs) != ctx.world_size:
            raise ValueError("all_gather needs one output tensor per rank")
        return outs, dist.all_gather(outs, t, **_kw(ctx, plan))

    return run


def _b_reduce_scatter(plan, ctx, dist):
    op = _reduce_op(dist, plan.reduce_op)

    def run(inv):
        out = _need_tensor(inv, "reduce_scatter")
        if len(inv.input_tensors) != ctx.world_size:
            raise ValueError("reduce_scatter needs one input tensor per rank")
        return out, dist.reduce_scatter(out, list(inv.input_tensors), op=op, **_kw(ctx, plan))

    return run


def _b_all_to_all(plan, ctx, dist):
    def run(inv):
        if len(inv.input_tensors) != ctx.world_size or len(inv.output_tensors) != ctx.world_size:
            raise ValueError("all_to_all needs one input and one output tensor per rank")
        outs = list(inv.output_tensors)
        return outs, dist.all_to_all(outs, list(inv.input_tensors), **_kw(ctx, plan))

    return run


def _global_rank(ctx: CompileContext, dist: Any, group_rank: int) -> int:
    if ctx.process_group is None:
        return group_rank
    getter = getattr(dist, "get_global_rank", None)
    return int(getter(ctx.process_group, group_rank)) if callable(getter) else group_rank


def _b_broadcast(plan, ctx, dist):
    src = _global_rank(ctx, dist, plan.root)

    def run(inv):
        t = _need_tensor(inv, "broadcast")
        return t, dist.broadcast(t, src=src, **_kw(ctx, plan))

    return run


def _b_reduce(plan, ctx, dist):
    op = _reduce_op(dist, plan.reduce_op)
    dst = _global_rank(ctx, dist, plan.root)

    def run(inv):
        t = _need_tensor(inv, "reduce")
        return t, dist.reduce(t, dst=dst, op=op, **_kw(ctx, plan))

    return run


def _b_gather(plan, ctx, dist):
    dst = _global_rank(ctx, dist, plan.root)

    def run(inv):
        t = _need_tensor(inv, "gather")
        outs = None
        if ctx.rank == plan.root:
            outs = list(inv.output_tensors) or [t.new_empty(t.shape) for _ in range(ctx.world_size)]
            if len(outs) != ctx.world_size:
                raise ValueError("gather needs one output tensor per rank on the root")
        return outs, dist.gather(t, gather_list=outs, dst=dst, **_kw(ctx, plan))

    return run


def _b_scatter(plan, ctx, dist):
    src = _global_rank(ctx, dist, plan.root)

    def run(inv):
        out = _need_tensor(inv, "scatter")
        pieces = None
        if ctx.rank == plan.root:
            pieces = list(inv.input_tensors)
            if len(pieces) != ctx.world_size:
                raise ValueError("scatter needs one input tensor per rank on the root")
        return out, dist.scatter(out, scatter_list=pieces, src=src, **_kw(ctx, plan))

    return run


def _b_barrier(plan, ctx, dist):
    def run(inv):
        kw = _kw(ctx, plan)
        if ctx.device.startswith("cuda") and ":" in ctx.device:
            kw["device_ids"] = [int(ctx.device.split(":")[1])]
        return None, dist.barrier(**kw)

    return run


NATIVE_BUILDERS: dict[str, Callable] = {
    "all_reduce": _b_all_reduce, "all_gather": _b_all_gather, "reduce_scatter": _b_reduce_scatter,
    "all_to_all": _b_all_to_all, "broadcast": _b_broadcast, "reduce": _b_reduce, "gather": _b_gather,
    "scatter": _b_scatter, "barrier": _b_barrier,
}
NATIVE_COLLECTIVES = tuple(NATIVE_BUILDERS)

# the reference's builder names (ccdl_comm/cuda/native_collectives.py:116-330): `(plan, context, dist) -> operation`
build_native_all_reduce, build_native_all_gather, build_native_reduce_scatter = \
    _b_all_reduce, _b_all_gather, _b_reduce_scatter
build_native_all_to_all, build_native_broadcast, build_native_reduce = _b_all_to_all, _b_broadcast, _b_reduce
build_native_gather, build_native_scatter, build_native_barrier = _b_gather, _b_scatter, _b_barrier


class NativeCollectiveExecutor:
    def __init__(self, operation: Callable, execution_info: ExecutionInfo) -> None:
        if not callable(operation):
            raise TypeError("operation must be callable")
        if not isinstance(execution_info, ExecutionInfo):
            raise TypeError("execution_info must be an ExecutionInfo")
        self._operation = operation
        self.execution_info = execution_info
        self.execution_counters = ExecutionCounters()
        self.last_handle: object | None = None

    def run(self, value: object):
        self.execution_counters._record_run()
        inv = value if isinstance(value, NativeCollectiveInput) else NativeCollectiveInput(tensor=value)
        try:
            result, handle = self._operation(inv)
        except BaseException:
            self.execution_counters._record_failed()
            raise
        self.last_handle = handle
        keep = tuple(t for t in (inv.tensor, *inv.input_tensors, *inv.output_tensors) if t is not None)
        work = CompletionWork(result, handle=handle, resources=keep)
        return bind_execution_work(work, self.execution_info, self.execution_counters)


def compile_native_collective(plan: CommunicationPlan, context: CompileContext, *, dist: Any | None = None,
                              require_nccl: bool = False) -> NativeCollectiveExecutor:
    if not isinstance(plan, CommunicationPlan):
        raise TypeError("plan must be a CommunicationPlan")
    if not isinstance(context, CompileContext):
        raise TypeError("context must be a CompileContext")
    if plan.strategy != "native_nccl":
        raise ValueError("native collective compiler requires strategy='native_nccl'")
    builder = NATIVE_BUILDERS.get(plan.collective)
    if builder is None:
        raise ValueError(f"unsupported native collective: {plan.collective!r}")
    if plan.root >= context.world_size:
        raise ValueError(f"root must be smaller than world_size ({plan.root} >= {context.world_size})")
    active = dist if dist is not None else import_module("torch.distributed")
    if require_nccl:
        backend = str(active.get_backend(context.process_group)).lower()
        if "nccl" not in backend:
            from ..exceptions import UnsupportedCollective

            raise UnsupportedCollective(f"{plan.collective}:native_nccl", reason=f"process group backend is {backend}")
    nbytes = 1
    for dim in context.shape:
        nbytes *= dim
    nbytes *= {"fp16": 2, "bf16": 2, "fp32": 4}.get(context.dtype, 4)
    info = ExecutionInfo(
        requested_strategy="native_nccl", executed_strategy="native_nccl", backend=plan.backend, fallback_used=False,
        fallback_reason=None, stage_names=(plan.collective,), original_bytes=nbytes, compressed_bytes=nbytes,
        compression_ratio=1.0, workspace_cache_hit=False, async_capable=True, fast_path="cuda_native_nccl",
        details={"collective": plan.collective, "root": plan.root, "reduce_op": plan.reduce_op})
    return NativeCollectiveExecutor(builder(plan, context, active), info)


CudaNativeCollectiveExecutor = NativeCollectiveExecutor   # the reference's class name
