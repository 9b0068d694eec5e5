"""CUDA completion events, the shared communication stream and work factory.

Parity: ccdl_comm/communication/cuda_completion.py:17-273.  `create_work`
returns the native `CompressedWork` when the extension is loaded and falls
back to the Python `CompletionWork` otherwise (and says so in ExecutionInfo).
"""

from __future__ import annotations

import threading
from dataclasses import replace
from typing import Any, Callable, Sequence

from ..core.info import ExecutionInfo
from ..core.work import CompletionWork

_STREAMS: dict[int, Any] = {}
_STREAM_LOCK = threading.Lock()


class NoopCompletion:
    """Stands in for an event when the tensor is not on a CUDA device."""

    def query(self) -> bool:
        return True

    def wait(self) -> None:
        return None

    def wait_stream(self, stream: Any = None) -> None:
        return None

    def synchronize(self) -> None:
        return None


class CudaCompletion:
    """A recorded CUDA event; `wait()` makes the *current stream* wait, not the host."""

    def __init__(self, event: Any) -> None:
        self.event = event

    def query(self) -> bool:
        return bool(self.event.query())

    def wait(self) -> None:
        self.event.wait()

    def wait_stream(self, stream: Any = None) -> None:
        if stream is None:
            self.event.wait()
        else:
            stream.wait_event(self.event)

    def synchronize(self) -> None:
        self.event.synchronize()


def comm_stream(device=None):
    """One high-priority side stream per device, shared by the library."""

    import torch

    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    with _STREAM_LOCK:
        stream = _STREAMS.get(index)
        if stream is None:
            stream = torch.cuda.Stream(device=index, priority=-1)
            _STREAMS[index] = stream
        return stream


class CudaStreamWork:
    """`with CudaStreamWork(torch=torch, async_op=True) as work:` runs the body on the communication stream
    (ordered after the caller's current stream) and records an event when the body ends; `work.wait()` makes
    the caller's current stream wait for that event (and waits on `handle` first when one was given), without
    blocking the host.  With `async_op=False` the body runs on the current stream and is already ordered.
    Parity: ccdl_comm/communication/cuda_completion.py:70-119.
    """

    def __init__(self, *, torch: Any, async_op: bool = False, handle: Any | None = None) -> None:
        self.async_op, self.handle, self._torch = async_op, handle, torch
        cuda = torch.cuda
        self.stream = _shared_comm_stream(cuda) if async_op else cuda.current_stream()
        self._guard = cuda.stream(self.stream)
        self.event = None

    def __enter__(self) -> "CudaStreamWork":
        self.stream.wait_stream(self._torch.cuda.current_stream())
        self._guard.__enter__()
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> None:
        self._guard.__exit__(exc_type, exc_value, traceback)
        self.event = self._torch.cuda.Event()
        self.event.record(self.stream)
        if not self.async_op:
            self.event.wait()

    def wait(self) -> None:
        waiter = getattr(self.handle, "wait", None)
        if callable(waiter):
            waiter()
        if self.async_op and self.event is not None:
            self.event.wait()

    def query(self) -> bool:
        if not self.async_op:
            return True
        return bool(self.event.query()) if self.event is not None else False


_SHARED_COMM_STREAMS: dict[int, Any] = {}


def _shared_comm_stream(cuda: Any) -> Any:
    device = int(cuda.current_device())
    if device not in _SHARED_COMM_STREAMS:
        _SHARED_COMM_STREAMS[device] = cuda.Stream(device)
    return _SHARED_COMM_STREAMS[device]


class CudaCompletionManager:
    def __init__(self, *, extension_status=None, torch_module=None, torch_provider=None) -> None:
        """`torch_module` is the module itself, `torch_provider` a zero-argument callable that returns it (the
        reference's spelling, ccdl_comm/communication/cuda_completion.py:176-183); tests pass fakes either way."""

        self._status = extension_status
        self._torch = torch_module
        self._torch_provider = torch_provider

    def _t(self):
        if self._torch is None:
            if self._torch_provider is not None:
                self._torch = self._torch_provider()
            else:
                import torch

                self._torch = torch
        return self._torch

    def record_for(self, tensor: Any, stream: Any = None):
        if not bool(getattr(tensor, "is_cuda", False)):
            return NoopCompletion()
        torch = self._t()
        event = torch.cuda.Event()
        event.record(stream if stream is not None else torch.cuda.current_stream(tensor.device))
        return CudaCompletion(event)

    def comm_stream(self, tensor: Any = None):
        return comm_stream(getattr(tensor, "device", None))

    def create_work(self, result: Any, *, handle: Any = None, complete: Callable[[], Any] | None = None,
                    completion: Any = None, resources: Sequence[Any] = (),
                    execution_info: ExecutionInfo | None = None, execution_counters=None, status_host: int = 0):
        native = self._native_module()
        if native is not None and execution_counters is None:
            work = native.CompressedWork(result, handle, completion, list(resources), complete, status_host)
            return work
        if execution_info is not None and native is None:
            execution_info = replace(execution_info, fast_path="python_fallback")
        return CompletionWork(result, handle=handle, complete=complete, completion=completion,
                              resources=resources, execution_info=execution_info,
                              execution_counters=execution_counters)

    def create_stream_work(self, result: Any, *, stream: Any, resources: Sequence[Any] = (),
                           execution_info: ExecutionInfo | None = None, execution_counters=None):
        """Work that completes when everything enqueued on `stream` so far has run."""

        completion = self.record_for(result if hasattr(result, "is_cuda") else _first_tensor(resources), stream)
        return CompletionWork(result, completion=completion, resources=resources, execution_info=execution_info,
                              execution_counters=execution_counters)

    def _native_module(self):
        from ..ops.loader import load_cuda_extension

        status = self._status if self._status is not None else load_cuda_extension()
        module = status.module if status.available else None
        if module is None or getattr(module, "NATIVE_WORK_ABI_VERSION", None) != 1:
            return None
        return module


def _first_tensor(values: Sequence[Any]):
    for v in values:
        if hasattr(v, "is_cuda"):
            return v
    return None


def native_work_available(extension_status: Any) -> bool:
    """Whether the extension carries the native work executor (`CudaExecutor` / `CompressedWork`) with the
    ABI this package speaks (ccdl_comm/communication/cuda_completion.py:148-156)."""

    from ..abi import NATIVE_WORK_ABI_VERSION

    module = getattr(extension_status, "module", None)
    return bool(getattr(extension_status, "available", False) and module is not None
                and hasattr(module, "create_cuda_executor")
                and getattr(module, "NATIVE_WORK_ABI_VERSION", None) == NATIVE_WORK_ABI_VERSION)
