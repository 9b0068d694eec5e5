"""The top-level package exposes every public name of `ccdl_comm` (ccdl_comm/__init__.py:61-125), so that
`import lowbit_comm_b200 as ccdl_comm` is a drop-in for code written against the reference."""

import lowbit_comm_b200 as lbc

REFERENCE_PUBLIC_NAMES = (
    "AutoStrategySelector", "BackendCapabilities", "BackendKey", "BackendRegistrationError", "BackendRegistry",
    "CCDLCommunicationPlugin", "CCDLError", "CCDLUnavailableError", "CCDL_CORE_ABI", "CapabilityReport",
    "CollectiveWork", "CommunicationBackend", "CommunicationPlan", "CommunicationStage", "CompileCache",
    "CompileCacheKey", "CompileContext", "CompiledCommunicationPlan", "CompiledExecutor", "CompletionWork",
    "CompressionConfig", "ExecutionCounterSnapshot", "ExecutionCounters", "ExecutionInfo", "ImmediateWork",
    "Quantizer", "ReducedShard", "ResolvedPlan", "StrategyChoice", "TorchDistributedUnavailableError",
    "UnsupportedCollective", "WorkspacePolicy", "all_gather", "all_reduce", "all_to_all", "barrier", "broadcast",
    "compile", "compile_collective", "compile_dynamic_all_gather", "compile_qrecv", "compile_qsend",
    "compressed_all_gather", "compressed_all_gather_dynamic", "compressed_all_reduce",
    "compressed_hierarchical_all_reduce", "compressed_reduce_scatter", "compressed_reduce_scatter_shard",
    "dequantize_tensor", "detect", "estimate_quantized_size", "gather", "iqrecv", "iqsend", "native_collectives",
    "qall_gather_dyn", "qrecv", "qsend", "quantize_tensor", "reduce", "reduce_scatter", "resolve_plan", "scatter",
)


def test_every_reference_name_is_exported():
    missing = [n for n in REFERENCE_PUBLIC_NAMES if not hasattr(lbc, n)]
    assert missing == []
    assert set(REFERENCE_PUBLIC_NAMES) <= set(lbc.__all__)


def test_lazy_names_resolve_to_callables_or_classes():
    for n in REFERENCE_PUBLIC_NAMES:
        obj = getattr(lbc, n)
        assert callable(obj) or isinstance(obj, (str, int, tuple)), n
