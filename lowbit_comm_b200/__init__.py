"""lowbit_comm_b200: low-bit compressed collectives for data-parallel training on B200.

Public names follow the reference package `ccdl_comm` (ccdl_comm/__init__.py:61-125).
Importing this package never imports torch; attributes that need torch are
resolved lazily on first access.
"""

from __future__ import annotations

from importlib import import_module

from .abi import CCDL_CORE_ABI, NATIVE_WORK_ABI_VERSION
from .capability import CapabilityReport, detect
from .config import CompressionConfig
from .core import (AutoStrategySelector, BackendCapabilities, BackendKey, BackendRegistry, BoundCollectiveWork, ChunkPlan,
                   CollectiveWork, CommunicationBackend, CommunicationPlan, CommunicationStage, CompileCache,
                   CompileCacheKey, CompileContext, CompiledCommunicationPlan, CompiledExecutor, CompletionWork,
                   ExecutionCounters, ExecutionCounterSnapshot, ExecutionInfo, GroupShardPlan, ImmediateWork,
                   ReducedShard, ResolvedPlan, StrategyChoice, WorkspacePolicy, bind_execution_work, compile,
                   resolve_plan)
from .exceptions import (AsyncCommunicationError, BackendRegistrationError, CCDLError, CCDLUnavailableError,
                         DeviceWaitStatus, TorchDistributedUnavailableError, UnsupportedCollective)
from .plugin import CCDLCommunicationPlugin, PluginDecision

__version__ = "0.1.0"

# name -> module that defines it (all of these import torch)
_LAZY = {
    "quantize_tensor": ".ops.codec", "dequantize_tensor": ".ops.codec", "dequantize_reduce_tensors": ".ops.codec",
    "inplace_quantize_pack": ".ops.codec", "inplace_dequantize_reduce_mean": ".ops.codec",
    "inplace_dequantize_reduce_mean_update_error_feedback": ".ops.codec",
    "dequantize_reduce_update_error_feedback": ".ops.codec", "update_error_feedback_residual": ".ops.codec",
    "allocate_quantized_buffer": ".ops.codec", "allocate_dequantized_buffer": ".ops.codec",
    "estimate_quantized_size": ".ops.sizing", "QuantizationSizeEstimate": ".ops.sizing",
    "Quantizer": ".ops.quantizer",
    "ErrorFeedbackState": ".ops.error_feedback", "ErrorFeedbackPolicy": ".ops.error_feedback",
    "ErrorFeedbackDecision": ".ops.error_feedback",
    "quantize_tensor_fallback": ".ops.torch_fallback", "dequantize_tensor_fallback": ".ops.torch_fallback",
    "load_cuda_extension": ".ops.loader", "CudaExtensionStatus": ".ops.loader",
    "create_ddp_comm_hook": ".parallel.ddp_hook",
    "CompressedPayload": ".parallel.payload", "GatheredPayloads": ".parallel.payload",
    "compressed_all_reduce": ".parallel.collectives", "compressed_all_gather": ".parallel.collectives",
    "compressed_reduce_scatter": ".parallel.collectives", "compressed_reduce_scatter_shard": ".parallel.collectives",
    "compressed_hierarchical_all_reduce": ".parallel.collectives",
    "compressed_all_gather_dynamic": ".parallel.collectives", "qall_gather_dyn": ".parallel.collectives",
    "compile_dynamic_all_gather": ".parallel.collectives",
    "all_reduce": ".parallel.collectives", "all_gather": ".parallel.collectives",
    "reduce_scatter": ".parallel.collectives", "all_to_all": ".parallel.collectives",
    "broadcast": ".parallel.collectives", "reduce": ".parallel.collectives", "gather": ".parallel.collectives",
    "scatter": ".parallel.collectives", "barrier": ".parallel.collectives",
    "compile_collective": ".parallel.collectives", "native_collectives": ".parallel.collectives",
    "qsend": ".parallel.p2p", "qrecv": ".parallel.p2p", "iqsend": ".parallel.p2p", "iqrecv": ".parallel.p2p",
    "compile_qsend": ".parallel.p2p", "compile_qrecv": ".parallel.p2p", "PointToPointWork": ".parallel.p2p",
    "register_cuda_backends": ".parallel.backend_cuda", "CudaCommunicationBackend": ".parallel.backend_cuda",
    "CudaWorkspacePool": ".parallel.workspace", "PeerGroup": ".parallel.peer_memory",
    "FusedWorkspace": ".parallel.fused",
    "plan_ddp_compression_strategy": ".parallel.strategy", "plan_bucket_fusion": ".parallel.bucket_fusion",
    "make_torch_all_gather": ".parallel.torch_transport", "make_torch_all_reduce": ".parallel.torch_transport",
    "make_torch_compressed_reduce_scatter_shard": ".parallel.transports",
    "make_torch_compressed_reduce_scatter_all_gather": ".parallel.transports",
    "make_native_topology_all_reduce": ".parallel.transports",
    "make_native_topology_reduce_scatter_shard": ".parallel.transports",
    "make_torch_hierarchical_all_reduce": ".parallel.transports",
    "make_legacy_topology_all_reduce": ".parallel.transports",
    "make_schedule_all_reduce": ".parallel.schedule_executors",
    "make_schedule_reduce_scatter_shard": ".parallel.schedule_executors",
    "PipelinedRingExecutor": ".parallel.schedule_executors", "TreeExecutor": ".parallel.schedule_executors",
    "PairwiseExecutor": ".parallel.schedule_executors", "ButterflyExecutor": ".parallel.schedule_executors",
}


# whole modules under the name code written against the reference imports them by
_LAZY_MODULES = {"ccdl_cuda_ops": ".ops.native_ops", "native_ops": ".ops.native_ops"}


def __getattr__(name: str):
    if name in _LAZY_MODULES:
        value = import_module(_LAZY_MODULES[name], __name__)
        globals()[name] = value
        return value
    target = _LAZY.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(import_module(target, __name__), name)
    globals()[name] = value
    return value


__all__ = sorted([n for n in globals() if not n.startswith("_")] + list(_LAZY) + list(_LAZY_MODULES))
