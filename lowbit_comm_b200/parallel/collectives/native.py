"""Public shortcuts for the nine native collectives (parity: ccdl_comm/collectives/api.py:14-337).

Every function returns a `CollectiveWork`; pass `compiled_plan` to reuse a plan
made by `compile_collective` in steady state.
"""

from __future__ import annotations

from importlib import import_module
from typing import Any

from ...core.compiler import compile as compile_plan, normalize_dtype
from ...core.executor import CompiledCommunicationPlan
from ...core.plan import CommunicationPlan, CompileContext
from ...core.registry import BackendRegistry
from ..native_collectives import NATIVE_COLLECTIVES, NativeCollectiveInput


def native_collectives() -> tuple[str, ...]:
    return NATIVE_COLLECTIVES


def context_from_tensor(tensor: object | None, *, group: object | None = None, device: str | None = None,
                        dist: Any | None = None, torch: Any | None = None) -> CompileContext:
    d = dist if dist is not None else import_module("torch.distributed")
    rank = int(d.get_rank(group=group))
    world = int(d.get_world_size(group=group))
    where = device or str(getattr(tensor, "device", ""))
    if not where:
        t = torch if torch is not None else import_module("torch")
        where = f"cuda:{int(t.cuda.current_device())}" if t.cuda.is_available() else "cpu"
    arch = "unknown"
    if where.startswith("cuda"):
        try:
            t = torch if torch is not None else import_module("torch")
            major, minor = t.cuda.get_device_capability(where)
            arch = f"sm_{major}{minor}"
        except Exception:  # noqa: BLE001
            arch = "unknown"
    return CompileContext(rank=rank, world_size=world, device=where, shape=tuple(getattr(tensor, "shape", ())),
                          dtype=normalize_dtype(str(getattr(tensor, "dtype", "fp32"))), process_group=group,
                          device_architecture=arch)


def compile_collective(sample: object | None, *, collective: str, group: object | None = None, root: int = 0,
                       op: str = "sum", async_op: bool = False, plan: CommunicationPlan | None = None,
                       registry: BackendRegistry | None = None, device: str | None = None) -> CompiledCommunicationPlan:
    active = plan or CommunicationPlan(collective=collective, strategy="native_nccl", backend="cuda",
                                       output_layout="full", async_op=async_op, root=root, reduce_op=op)
    if active.collective != collective:
        raise ValueError(f"plan collective {active.collective!r} does not match requested collective {collective!r}")
    context = context_from_tensor(sample, group=group, device=device)
    reg = registry
    if reg is None:
        from ..backend_cuda import register_cuda_backends

        reg = BackendRegistry()
        register_cuda_backends(reg, allow_cpu=not context.device.startswith("cuda"))
    return compile_plan(active, context, registry=reg)


def _run(sample, invocation, *, collective, group, root=0, op="sum", async_op=False, plan=None, compiled_plan=None,
         device=None):
    compiled = compiled_plan or compile_collective(sample, collective=collective, group=group, root=root, op=op,
                                                   async_op=async_op, plan=plan, device=device)
    work = compiled.run(invocation)
    if not async_op and compiled_plan is None:
        work.wait()
    return work


def all_reduce(tensor, *, op="sum", group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(tensor, tensor, collective="all_reduce", group=group, op=op, async_op=async_op, plan=plan,
                compiled_plan=compiled_plan)


def all_gather(tensor, *, output_tensors=(), group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(tensor, NativeCollectiveInput(tensor=tensor, output_tensors=tuple(output_tensors)),
                collective="all_gather", group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def reduce_scatter(output, *, input_tensors, op="sum", group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(output, NativeCollectiveInput(tensor=output, input_tensors=tuple(input_tensors)),
                collective="reduce_scatter", group=group, op=op, async_op=async_op, plan=plan,
                compiled_plan=compiled_plan)


def all_to_all(*, output_tensors, input_tensors, group=None, async_op=False, plan=None, compiled_plan=None):
    sample = input_tensors[0] if input_tensors else None
    return _run(sample, NativeCollectiveInput(input_tensors=tuple(input_tensors), output_tensors=tuple(output_tensors)),
                collective="all_to_all", group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def broadcast(tensor, *, src=0, group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(tensor, tensor, collective="broadcast", group=group, root=src, async_op=async_op, plan=plan,
                compiled_plan=compiled_plan)


def reduce(tensor, *, dst=0, op="sum", group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(tensor, tensor, collective="reduce", group=group, root=dst, op=op, async_op=async_op, plan=plan,
                compiled_plan=compiled_plan)


def gather(tensor, *, gather_list=(), dst=0, group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(tensor, NativeCollectiveInput(tensor=tensor, output_tensors=tuple(gather_list)), collective="gather",
                group=group, root=dst, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def scatter(output, *, scatter_list=(), src=0, group=None, async_op=False, plan=None, compiled_plan=None):
    return _run(output, NativeCollectiveInput(tensor=output, input_tensors=tuple(scatter_list)), collective="scatter",
                group=group, root=src, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def barrier(*, group=None, async_op=False, device=None, plan=None, compiled_plan=None):
    return _run(None, NativeCollectiveInput(), collective="barrier", group=group, async_op=async_op, plan=plan,
                compiled_plan=compiled_plan, device=device)
