"""The nine uncompressed collectives behind the same compile/run interface as the compressed ones.

`lbc.all_reduce(t)`, `lbc.broadcast(t, src=1)` ... each describe their call as a `_Call` (which tensor stands
for the shape, what is handed to the executor, who is root) and `_Call.submit` does the rest: compile -- or take
the caller's `compiled_plan` -- run, and for a synchronous one-off call wait.  One-off calls compile against
one process-wide default registry per device kind and through a small LRU of compiled plans, so a loop that
calls `lbc.all_reduce(t)` with the same shape compiles once.  Every function returns a `CollectiveWork`.
Names and keyword arguments are the reference's (ccdl_comm/collectives/api.py:14-337).
"""

from __future__ import annotations

from dataclasses import dataclass
from importlib import import_module
from typing import Any

from ...core.compiler import CompileCache, compile as compile_plan, normalize_dtype
from ...core.executor import CompiledCommunicationPlan
from ...core.plan import CommunicationPlan, CompileContext
from ...core.registry import BackendRegistry
from ..native_collectives import NATIVE_COLLECTIVES, NativeCollectiveInput

_default_registries: dict[bool, BackendRegistry] = {}
_one_off_plans = CompileCache(max_entries=32)


def native_collectives() -> tuple[str, ...]:
    return NATIVE_COLLECTIVES


def _default_registry(on_cuda: bool) -> BackendRegistry:
    registry = _default_registries.get(on_cuda)
    if registry is None:
        from ..backend_cuda import register_cuda_backends

        registry = BackendRegistry()
        register_cuda_backends(registry, allow_cpu=not on_cuda)
        _default_registries[on_cuda] = registry
    return registry


def _architecture(device: str, torch: Any | None) -> str:
    """`sm_<major><minor>` of a CUDA device, "unknown" for anything else or when it cannot be asked."""

    if not device.startswith("cuda"):
        return "unknown"
    try:
        major, minor = (torch or import_module("torch")).cuda.get_device_capability(device)
    except Exception:  # noqa: BLE001  (no torch, no driver, bad index: the fact is simply not known)
        return "unknown"
    return f"sm_{major}{minor}"


def context_from_tensor(tensor: object | None, *, group: object | None = None, device: str | None = None,
                        dist: Any | None = None, torch: Any | None = None) -> CompileContext:
    """Compile-time facts read off one representative tensor and the process group.  Without a tensor and
    without `device`, the current CUDA device is meant when there is one, else the CPU."""

    dist = dist or import_module("torch.distributed")
    where = device or str(getattr(tensor, "device", ""))
    if not where:
        cuda = (torch or import_module("torch")).cuda
        where = f"cuda:{int(cuda.current_device())}" if cuda.is_available() else "cpu"
    return CompileContext(
        rank=int(dist.get_rank(group=group)), world_size=int(dist.get_world_size(group=group)), device=where,
        shape=tuple(getattr(tensor, "shape", ())), dtype=normalize_dtype(str(getattr(tensor, "dtype", "fp32"))),
        process_group=group, device_architecture=_architecture(where, torch))


def compile_collective(sample: object | None, *, collective: str, group: object | None = None, root: int = 0,
                       op: str = "sum", async_op: bool = False, plan: CommunicationPlan | None = None,
                       registry: BackendRegistry | None = None, device: str | None = None,
                       cache: CompileCache | None = None) -> CompiledCommunicationPlan:
    """A reusable plan for one native collective on tensors shaped like `sample`."""

    if plan is None:
        plan = CommunicationPlan(collective=collective, strategy="native_nccl", backend="cuda", output_layout="full",
                                 async_op=async_op, root=root, reduce_op=op)
    elif plan.collective != collective:
        raise ValueError(f"plan collective {plan.collective!r} does not match requested collective {collective!r}")
    context = context_from_tensor(sample, group=group, device=device)
    return compile_plan(plan, context, cache=cache,
                        registry=registry or _default_registry(context.device.startswith("cuda")))


@dataclass(frozen=True)
class _Call:
    collective: str
    sample: object | None          # stands for shape, dtype and device at compile time
    payload: object                # what the executor's run() receives
    root: int = 0
    op: str = "sum"

    def submit(self, *, group, async_op, plan, compiled_plan, device=None):
        if compiled_plan is not None:
            return compiled_plan.run(self.payload)
        work = compile_collective(self.sample, collective=self.collective, group=group, root=self.root, op=self.op,
                                  async_op=async_op, plan=plan, device=device, cache=_one_off_plans).run(self.payload)
        if not async_op:
            work.wait()
        return work


def _lists(tensor=None, *, inputs=(), outputs=()) -> NativeCollectiveInput:
    return NativeCollectiveInput(tensor=tensor, input_tensors=tuple(inputs), output_tensors=tuple(outputs))


def all_reduce(tensor, *, op="sum", group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("all_reduce", tensor, tensor, op=op)
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def broadcast(tensor, *, src=0, group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("broadcast", tensor, tensor, root=src)
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def reduce(tensor, *, dst=0, op="sum", group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("reduce", tensor, tensor, root=dst, op=op)
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def all_gather(tensor, *, output_tensors=(), group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("all_gather", tensor, _lists(tensor, outputs=output_tensors))
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def gather(tensor, *, gather_list=(), dst=0, group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("gather", tensor, _lists(tensor, outputs=gather_list), root=dst)
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def reduce_scatter(output, *, input_tensors, op="sum", group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("reduce_scatter", output, _lists(output, inputs=input_tensors), op=op)
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def scatter(output, *, scatter_list=(), src=0, group=None, async_op=False, plan=None, compiled_plan=None):
    call = _Call("scatter", output, _lists(output, inputs=scatter_list), root=src)
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def all_to_all(*, output_tensors, input_tensors, group=None, async_op=False, plan=None, compiled_plan=None):
    both = (*input_tensors, *output_tensors)
    if not both:
        raise ValueError("all_to_all requires at least one tensor")
    call = _Call("all_to_all", both[0], _lists(inputs=input_tensors, outputs=output_tensors))
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan)


def barrier(*, group=None, async_op=False, device=None, plan=None, compiled_plan=None):
    call = _Call("barrier", None, _lists())
    return call.submit(group=group, async_op=async_op, plan=plan, compiled_plan=compiled_plan, device=device)
