"""The single compute backend behind the compile-once control plane.

Parity: ccdl_comm/cuda/backend.py:23-253 (`CudaCommunicationBackend`,
`register_cuda_backends`, capability report), ccdl_comm/cuda/compiler.py:82-865
(binding a plan to an operation and an `ExecutionInfo`), ccdl_comm/cuda/
executors.py:30-220 (`CudaAllReduceExecutor`, `CompressedReduceScatterExecutor`
with output leases) and ccdl_comm/cuda/shortcut.py:18-59 (one-shot compile; here
with a cache instead of a fresh registry per call).

Everything a `run()` needs is resolved in `compile()`: the communicator of the
process group, the strategy (stage count), the reduce scale, the workspace key.
`run()` only validates the tensor against the compiled shape and enqueues kernels.
"""

from __future__ import annotations

import threading
from collections.abc import Callable, Mapping
from dataclasses import dataclass, replace
from typing import Any

from ..config import CompressionConfig
from ..core.backend import BackendCapabilities
from ..core.compiler import CompileCache, compile as compile_plan, normalize_dtype
from ..core.executor import CompiledCommunicationPlan
from ..core.info import ExecutionCounters, ExecutionInfo
from ..core.plan import CommunicationPlan, CompileContext
from ..core.registry import BackendKey, BackendRegistry
from ..core.work import bind_execution_work
from ..exceptions import UnsupportedCollective
from ..ops.loader import CudaExtensionStatus, load_cuda_extension
from ..ops.sizing import estimate_quantized_size
from .native_collectives import NATIVE_COLLECTIVES, compile_native_collective
from .strategy_table import CudaStrategyTable
from .workspace import CudaOutputLease, CudaWorkspacePool, WorkspaceKey

OperationKey = tuple[str, str, str]
CUDA_BACKEND_KEYS: tuple[OperationKey, ...] = (
    *((name, "native_nccl", "full") for name in NATIVE_COLLECTIVES),
    ("all_reduce", "all_gather", "full"),
    ("all_reduce", "reduce_scatter", "full"),
    ("all_reduce", "topology", "full"),
    ("all_reduce", "hierarchical", "full"),
    ("all_gather", "compressed", "full"),
    ("reduce_scatter", "compressed", "shard"),
)
_FAST_PATH = {"all_gather": "cuda_fused_one_stage", "reduce_scatter": "cuda_fused_two_stage",
              "topology": "cuda_fused_two_stage", "hierarchical": "cuda_hierarchical",
              "compressed": "cuda_reduced_shard"}


def _numel(shape) -> int:
    total = 1
    for d in shape:
        total *= d
    return total


def _check_tensor(tensor: Any, context: CompileContext) -> None:
    if tuple(getattr(tensor, "shape", ())) != tuple(context.shape):
        raise ValueError(f"tensor shape {tuple(tensor.shape)} does not match the compiled shape {context.shape}")
    if normalize_dtype(str(tensor.dtype)) != normalize_dtype(context.dtype):
        raise TypeError(f"tensor dtype {tensor.dtype} does not match the compiled dtype {context.dtype}")


def _tensor_checker(context: CompileContext) -> Callable[[Any], None]:
    """`_check_tensor` for a hot path: the shape is compared as a tuple prepared once, and a dtype object that
    passed before is recognised by identity instead of being turned into a name again."""

    want_shape = tuple(context.shape)
    passed: list[Any] = [None]

    def check(tensor: Any) -> None:
        if tensor.shape != want_shape or tensor.dtype is not passed[0]:
            _check_tensor(tensor, context)
            passed[0] = tensor.dtype

    return check


def _reason_iff_negative(flag: bool, reason: str | None, *, what: str, positive: str) -> None:
    """A record that says "yes" carries no explanation, one that says "no" must say why."""

    if flag and reason is not None:
        raise ValueError(f"{what}: {positive}, so there is nothing to explain (got reason {reason!r})")
    if not flag and not (isinstance(reason, str) and reason.strip()):
        raise ValueError(f"{what}: not {positive}, so the reason has to be stated")


@dataclass(frozen=True)
class PrecollectedPayloadExecution:
    """What reducing already-gathered payloads did: where the result is, and whether the fused
    decode + mean (+ residual) kernel served it or why not (ccdl_comm/cuda/executors.py:16-27)."""

    output: object
    fused: bool
    fallback_reason: str | None = None

    def __post_init__(self) -> None:
        _reason_iff_negative(self.fused, self.fallback_reason, what="precollected-payload execution",
                             positive="served by the fused kernel")


@dataclass(frozen=True)
class FusedReducedShardCapability:
    """Compile-time answer to "can this reduce-scatter hand out its shard through the fused kernels?"
    (ccdl_comm/cuda/compiler.py:69-79)."""

    available: bool
    reason: str | None = None

    def __post_init__(self) -> None:
        _reason_iff_negative(self.available, self.reason, what="fused reduced-shard capability",
                             positive="available")


def fused_reduced_shard_capability(plan: CommunicationPlan, context: CompileContext,
                                   *, peer_access: bool) -> FusedReducedShardCapability:
    """The fused scatter + reduce kernels serve linear profiles without top-k on CUDA tensors of ranks with
    peer access; everything else goes through the all-to-all staging of torch.distributed."""

    from ..ops import codec

    if not str(context.device).startswith("cuda"):
        return FusedReducedShardCapability(False, f"device {context.device!r} has no peer-memory path")
    if plan.compression is None or not codec.is_fast_profile(plan.compression):
        return FusedReducedShardCapability(False, "the compression profile needs the general codec kernels")
    if not peer_access:
        return FusedReducedShardCapability(False, "no peer access between the ranks of this group")
    return FusedReducedShardCapability(True)


class CudaAllReduceExecutor:
    """Runs one precompiled compressed all-reduce (or all-gather) operation."""

    def __init__(self, operation: Callable[[Any], Any], execution_info: ExecutionInfo, *,
                 precollected: Callable[..., Any] | None = None,
                 precollected_operation: Callable[..., Any] | None = None) -> None:
        """`precollected(payloads, prepared, output, residual)` serves `run_precollected_payloads`;
        `precollected_operation` is the reference's name for the same argument."""

        if not callable(operation):
            raise TypeError("operation must be callable")
        if not isinstance(execution_info, ExecutionInfo):
            raise TypeError("execution_info must be an ExecutionInfo")
        self._operation = operation
        self._precollected = precollected if precollected is not None else precollected_operation
        self.execution_info = execution_info
        self.last_execution_info = execution_info      # what the most recent precollected run actually did
        self.execution_counters = ExecutionCounters()

    def run(self, tensor: Any):
        self.execution_counters._record_run()
        try:
            result = self._operation(tensor)
        except BaseException:
            self.execution_counters._record_failed()
            raise
        return bind_execution_work(result, self.execution_info, self.execution_counters)

    def run_precollected_payloads(self, payloads, prepared, output, residual=None):
        """DDP fast path: the payloads are already gathered; fuse decode + mean (+ residual update)."""

        if self._precollected is None:
            raise UnsupportedCollective("all_reduce:precollected", reason="operation has no precollected path")
        self.execution_counters._record_run()
        try:
            result = self._precollected(payloads, prepared, output, residual)
        except BaseException:
            self.execution_counters._record_failed()
            raise
        info = self.execution_info
        if isinstance(result, PrecollectedPayloadExecution):
            if result.fused:
                info = replace(info, fallback_used=False, fallback_reason=None,
                               fast_path="cuda_fused_dequant_reduce_mean_ef")
            else:
                info = replace(info, fallback_used=True, fallback_reason=result.fallback_reason,
                               fast_path="per_payload_decode")
            result = result.output
        self.last_execution_info = info
        return bind_execution_work(result, info, self.execution_counters)


class CompressedReduceScatterExecutor:
    """Reduced-shard executor with pooled, lease-managed outputs."""

    def __init__(self, operation: Callable[..., Any], execution_info: ExecutionInfo, *, shard_numel: int,
                 pool: CudaWorkspacePool, key: WorkspaceKey, completion_manager: Any, stream_provider: Callable[[], Any]):
        self._operation = operation
        self.execution_info = execution_info
        self.execution_counters = ExecutionCounters()
        self.shard_numel = shard_numel
        self._pool, self._key, self._manager, self._stream = pool, key, completion_manager, stream_provider
        self._token = object()

    @property
    def workspace_stats(self):
        return self._pool.stats

    def acquire_output(self) -> CudaOutputLease:
        stream = self._stream()
        return CudaOutputLease(self._pool.acquire(self._key, stream), owner_token=self._token,
                               completion_manager=self._manager, acquisition_stream=stream)

    def run(self, tensor: Any, *, out: Any = None):
        self.execution_counters._record_run()
        lease = out if isinstance(out, CudaOutputLease) else None
        try:
            target = lease.mark_used(self._token) if lease is not None else out
            result = self._operation(tensor, target)
        except BaseException:
            if lease is not None and lease.state == "SUBMITTING":
                lease.abort_use(self._token)
            self.execution_counters._record_failed()
            raise
        work = bind_execution_work(result, self.execution_info, self.execution_counters)
        if lease is not None:
            lease.bind_work(self._token, work)
        return work


CudaReducedShardExecutor = CompressedReduceScatterExecutor


class CudaCommunicationBackend:
    name = "cuda"
    abi_version = 1

    def __init__(self, *, extension_status: CudaExtensionStatus | None = None,
                 operation_factories: Mapping[OperationKey, Callable] | None = None,
                 communicator_factory: Callable[[Any], Any] | None = None, allow_cpu: bool = False,
                 name: str | None = None) -> None:
        self._status = extension_status or load_cuda_extension()
        self._keys = tuple(operation_factories) if operation_factories is not None else CUDA_BACKEND_KEYS
        self._factories = dict(operation_factories or {})
        self._communicator_factory = communicator_factory
        self._allow_cpu = allow_cpu
        if name is not None:
            self.name = name

    # -- capabilities ---------------------------------------------------------
    def capabilities(self, context: CompileContext) -> BackendCapabilities:
        keys = [k for k in self._keys if k[1] != "hierarchical" or _hierarchical_possible(context)]
        native_only = bool(keys) and all(k[1] == "native_nccl" for k in keys)
        on_cuda = context.device.strip().lower().startswith("cuda")
        ext_ok = self._status.available and self._status.module is not None
        available, reason = True, None
        if not on_cuda and not self._allow_cpu:
            available, reason = False, f"device {context.device!r} is not CUDA"
        elif on_cuda and not native_only and not ext_ok:
            available, reason = False, self._status.reason or "sm_100a extension is unavailable"
        features = {"compile_once"}
        features.add("native_nccl" if native_only else "workspace_cache")
        if ext_ok:
            features.update({"cuda_extension", "fused_peer_collectives"})
        return BackendCapabilities(
            backend=self.name, available=available, collectives={k[0] for k in keys}, strategies={k[1] for k in keys},
            dtypes={"fp16", "bf16", "fp32"}, bits={4, 8}, output_layouts={k[2] for k in keys}, supports_async=True,
            supports_dynamic_shape=False, features=features, reason=reason,
            details={"abi_version": self.abi_version, "architecture": "sm_100a"})

    # -- compile ----------------------------------------------------------------
    def compile(self, plan: CommunicationPlan, context: CompileContext):
        key = (plan.collective, plan.strategy, plan.output_layout)
        if key not in self._keys:
            raise UnsupportedCollective(":".join(key), reason="operation is not provided by this backend")
        if key in self._factories:
            return self._factories[key](plan, context)
        if plan.strategy == "native_nccl":
            return compile_native_collective(plan, context)
        if plan.compression is None:
            raise UnsupportedCollective(":".join(key), reason="a CompressionConfig is required")
        if plan.reduce_op not in ("mean", "sum") and plan.collective != "all_gather":
            raise UnsupportedCollective(":".join(key), reason="only reduce_op 'mean' and 'sum' are implemented")
        comm = self._communicator(context)
        info = self._info(plan, context)
        cfg, op, dtype = plan.compression, plan.reduce_op, normalize_dtype(context.dtype)
        if plan.collective == "all_reduce" and plan.strategy == "hierarchical" and plan.stages:
            return CudaAllReduceExecutor(self._staged_hierarchy(plan, context, dtype), info)
        if plan.collective == "all_reduce":
            strategy = plan.strategy
            check = _tensor_checker(context)
            if plan.async_op:
                def operation(tensor):
                    check(tensor)
                    return comm.all_reduce(tensor, config=cfg, op=op, strategy=strategy, async_op=True, dtype=dtype)
            else:
                # compile once: the workspace and the stage count are bound here, not looked up per call
                bound = comm.bind_all_reduce(config=cfg, op=op, strategy=strategy, dtype=dtype)

                def operation(tensor):
                    check(tensor)
                    return bound(tensor)

            def precollected(payloads, prepared, output, residual):
                from ..ops import codec

                if residual is not None:
                    fused = codec.inplace_dequantize_reduce_mean_update_error_feedback(
                        payloads, prepared, output, residual, cfg, reduce=op)
                else:
                    fused = codec.inplace_dequantize_reduce_mean(payloads, output, cfg, reduce=op)
                if fused:
                    return PrecollectedPayloadExecution(output, True)
                # profiles or payload counts the fused kernel does not take: decode payload by payload
                codec.dequantize_reduce_tensors(payloads, tuple(output.shape), cfg, dtype=dtype, output=output, reduce=op)
                if residual is not None:
                    codec.update_error_feedback_residual(prepared, output, residual)
                return PrecollectedPayloadExecution(output, False, "profile or payload count outside the fused "
                                                                   "decode-reduce kernel")

            return CudaAllReduceExecutor(operation, info, precollected=precollected)
        if plan.collective == "all_gather":
            def gather_operation(tensor):
                _check_tensor(tensor, context)
                return comm.all_gather(tensor, config=cfg, async_op=plan.async_op, dtype=dtype)

            return CudaAllReduceExecutor(gather_operation, info)
        # reduce_scatter / compressed / shard
        from .completion import CudaCompletionManager
        from .fused import geometry

        n = _numel(context.shape)
        shard_numel = geometry(n, context.world_size, dtype, cfg).shard_numel
        pool = CudaWorkspacePool(allocator=_shard_allocator(context.device, dtype),
                                 max_cached_bytes=plan.workspace_policy.max_cached_bytes,
                                 max_entries=plan.workspace_policy.max_entries)
        wkey = WorkspaceKey(backend=self.name, collective="reduce_scatter", strategy="compressed",
                            shape_class=(shard_numel,), dtype=dtype, world_size=context.world_size, bit=cfg.bit,
                            group_size=cfg.group_size, chunk_config=(shard_numel,), workspace_kind="reduced_output",
                            device=context.device)

        def shard_operation(tensor, out):
            _check_tensor(tensor, context)
            return comm.reduce_scatter_shard(tensor, config=cfg, op=op, async_op=plan.async_op, dtype=dtype, out=out)

        return CompressedReduceScatterExecutor(shard_operation, info, shard_numel=shard_numel, pool=pool, key=wkey,
                                               completion_manager=CudaCompletionManager(extension_status=self._status),
                                               stream_provider=_current_stream_provider(context.device))

    def _staged_hierarchy(self, plan: CommunicationPlan, context: CompileContext, dtype: str):
        """A plan that spells out its three stages is compiled stage by stage (`core/hierarchy.py`); every stage
        runs on the communicator of its own process group: fused kernels inside the local group for the
        reduce-scatter and the gather, a compressed all-reduce of the shard between the groups."""

        from importlib import import_module

        from ..core.hierarchy import compile_hierarchical_stages

        torch = import_module("torch")
        dist = import_module("torch.distributed")
        n = _numel(context.shape)
        op = plan.reduce_op

        def bind(stage, stage_context):
            comm = self._communicator(stage_context)
            cfg = stage.compression or plan.compression
            if stage.collective == "reduce_scatter":
                return lambda tensor: comm.reduce_scatter_shard(tensor, config=cfg, op=op, dtype=dtype).shard
            if stage.collective == "all_reduce":
                strategy = "auto" if stage.strategy in ("topology", "compressed") else stage.strategy

                def inter(piece):
                    if comm.world_size == 1:
                        return piece
                    return comm.all_reduce(piece, config=cfg, op=op, strategy=strategy, dtype=dtype)

                return inter

            def gather(piece):
                if stage.strategy == "native_nccl":
                    parts = [torch.empty_like(piece) for _ in range(comm.world_size)]
                    kw = {} if stage_context.process_group is None else {"group": stage_context.process_group}
                    dist.all_gather(parts, piece.contiguous(), **kw)
                else:
                    parts = comm.all_gather(piece, config=cfg, dtype=dtype)
                return torch.cat([p.reshape(-1) for p in parts])[:n].reshape(context.shape)

            return gather

        chain = compile_hierarchical_stages(plan, context, operation_factory=bind,
                                            group_factory=lambda ranks: dist.new_group(list(ranks)))

        def operation(tensor):
            _check_tensor(tensor, context)
            work = chain.run(tensor)
            return work if plan.async_op else work.wait()

        return operation

    def _communicator(self, context: CompileContext):
        if self._communicator_factory is not None:
            return self._communicator_factory(context.process_group)
        from .communicator import get_communicator

        return get_communicator(context.process_group)

    def _info(self, plan: CommunicationPlan, context: CompileContext) -> ExecutionInfo:
        dtype = normalize_dtype(context.dtype)
        n = _numel(context.shape)
        est = estimate_quantized_size(n, dtype=dtype, config=plan.compression)
        on_cuda = context.device.lower().startswith("cuda")
        return ExecutionInfo(
            requested_strategy=plan.strategy, executed_strategy=plan.strategy, backend=self.name, fallback_used=False,
            fallback_reason=None, stage_names=tuple(s.name for s in plan.stages) or (plan.collective,),
            original_bytes=est.original_bytes, compressed_bytes=max(est.quantized_bytes, 0),
            compression_ratio=est.compression_ratio if est.quantized_bytes else 1.0, workspace_cache_hit=False,
            async_capable=True, fast_path=_FAST_PATH.get(plan.strategy, "cuda_fused") if on_cuda else "torch_fallback",
            details={"world_size": context.world_size, "bit": plan.compression.bit,
                     "group_size": plan.compression.group_size, "reduce_op": plan.reduce_op,
                     "peer_memory": on_cuda})


def _hierarchical_possible(context: CompileContext) -> bool:
    local = context.local_world_size
    return context.world_size >= 2 and (local is None or (0 < local <= context.world_size
                                                          and context.world_size % local == 0))


def _shard_allocator(device: str, dtype: str):
    def allocate(key: WorkspaceKey, stream: Any):
        import torch

        from ..ops.oracle import TORCH_DTYPES

        return torch.empty(key.shape_class, dtype=TORCH_DTYPES[dtype], device=device)

    return allocate


def _current_stream_provider(device: str):
    def provide():
        if not device.lower().startswith("cuda"):
            return None
        import torch

        return torch.cuda.current_stream(device)

    return provide


def register_cuda_backends(registry: BackendRegistry, *, extension_status: CudaExtensionStatus | None = None,
                           operation_factories: Mapping[OperationKey, Callable] | None = None,
                           allow_cpu: bool = False, backend_name: str = "cuda",
                           strategy_table: CudaStrategyTable | None = None) -> None:
    """Register every (collective, strategy, layout) key of the backend plus its auto-strategy table."""

    keys = tuple(operation_factories) if operation_factories is not None else CUDA_BACKEND_KEYS

    def factory():
        return CudaCommunicationBackend(extension_status=extension_status, operation_factories=operation_factories,
                                        allow_cpu=allow_cpu, name=backend_name)

    for collective, strategy, layout in keys:
        registry.register(BackendKey(collective, strategy, backend_name, layout), factory)
    if registry.strategy_selector(backend_name) is None:
        registry.register_strategy_selector(backend_name, (strategy_table or CudaStrategyTable.for_b200()).as_selector())


def default_operation_factories() -> dict[OperationKey, Callable | None]:
    """The (collective, strategy, output layout) keys the CUDA backend serves out of the box.  The reference
    maps each key to a host-side operation builder (ccdl_comm/cuda/compiler.py:122-146); here one backend
    object compiles all of them onto the communicator, so the values are None: a placeholder that callers
    override per key to inject their own builder `(plan, context) -> executor`."""

    return {key: None for key in CUDA_BACKEND_KEYS}


def compile_cuda_plan(plan: CommunicationPlan, context: CompileContext,
                      extension_status: CudaExtensionStatus | None = None, *,
                      operation_factories: Mapping[OperationKey, Callable] | None = None, allow_cpu: bool = False):
    """Compile one validated plan straight with the CUDA backend, without a registry
    (ccdl_comm/cuda/compiler.py:82-119).  Entries of `operation_factories` that are None keep the built-in path."""

    given = None
    if operation_factories is not None:
        given = {k: v for k, v in operation_factories.items() if v is not None} or None
    backend = CudaCommunicationBackend(extension_status=extension_status, operation_factories=given,
                                       allow_cpu=allow_cpu)
    if given is not None:                      # injected builders add to the built-in keys, they do not replace them
        backend._keys = tuple(dict.fromkeys((*CUDA_BACKEND_KEYS, *given)))
    return backend.compile(plan, context)


_SHORTCUT_LOCK = threading.Lock()
_SHORTCUT_REGISTRIES: dict[tuple, BackendRegistry] = {}
_SHORTCUT_CACHE = CompileCache(max_entries=256)


def compile_cuda_shortcut(tensor: Any, *, collective: str, strategy: str, output_layout: str,
                          config: CompressionConfig | None, async_op: bool = False, dtype: str = "auto",
                          extension_status: CudaExtensionStatus | None = None, group: Any = None,
                          reduce_op: str = "mean") -> CompiledCommunicationPlan:
    """Compile (and cache) a plan for `tensor`'s shape on the calling rank."""

    from .collectives.native import context_from_tensor

    context = context_from_tensor(tensor, group=group)
    on_cpu = not context.device.startswith("cuda")
    with _SHORTCUT_LOCK:
        reg_key = (id(extension_status), on_cpu)
        registry = _SHORTCUT_REGISTRIES.get(reg_key)
        if registry is None:
            registry = BackendRegistry()
            register_cuda_backends(registry, extension_status=extension_status, allow_cpu=on_cpu)
            _SHORTCUT_REGISTRIES[reg_key] = registry
    plan = CommunicationPlan(collective=collective, strategy=strategy, backend="cuda", compression=config,
                             output_layout=output_layout, async_op=async_op, reduce_op=reduce_op)
    if dtype != "auto":
        from dataclasses import replace

        context = replace(context, dtype=dtype)
    return compile_plan(plan, context, registry=registry, cache=_SHORTCUT_CACHE)
