"""Transports over `torch.distributed` (NCCL on GPUs, gloo on CPUs).

Role parity: ccdl_comm/communication/torch_transport.py:61-188.  These are the
fallback and baseline transports: a payload is an opaque tensor moved by a
library collective.  On one NVLink domain the fused peer-memory kernels replace
them; they remain the path for CPU/gloo runs, multi-node groups and the
generic-codec configurations.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from importlib import import_module as _std_import
from typing import Any

from ..exceptions import TorchDistributedUnavailableError
from .payload import CompressedPayload, GatheredPayloads, payload_buffer


def _dist(importer: Callable[[str], Any]):
    try:
        dist = importer("torch.distributed")
    except (ImportError, ModuleNotFoundError) as exc:
        raise TorchDistributedUnavailableError("torch.distributed is not available") from exc
    if not dist.is_available() or not dist.is_initialized():
        raise TorchDistributedUnavailableError("torch.distributed is not initialized")
    return dist


def _op(dist, name: str):
    key = name.strip().upper()
    table = getattr(dist, "ReduceOp", None)
    if table is None or not hasattr(table, key):
        raise ValueError(f"unsupported torch.distributed reduce op: {name}")
    return getattr(table, key)


def _group_kw(group) -> dict:
    return {} if group is None else {"group": group}


def _world(dist, group) -> int:
    return int(dist.get_world_size(group)) if group is not None else int(dist.get_world_size())


class HandleWork:
    """A c10d handle plus the value its completion makes valid."""

    def __init__(self, handle: Any, value: Any) -> None:
        self.handle, self.value = handle, value

    def wait(self) -> Any:
        self.handle.wait()
        return self.value

    def is_completed(self) -> bool:
        probe = getattr(self.handle, "is_completed", None)
        return bool(probe()) if callable(probe) else False

    def get_future(self) -> Any:
        getter = getattr(self.handle, "get_future", None)
        return getter() if callable(getter) else None


# Names the reference exports for the same roles.
AsyncAllGatherWork = HandleWork
AsyncAllReduceWork = HandleWork


def make_torch_all_reduce(*, group=None, import_module=_std_import) -> Callable[[CompressedPayload, str], CompressedPayload]:
    """Byte-wise all-reduce of the payload buffer.

    Kept for API parity only: summing int8 codes and scales as bytes is not a
    valid reduction for world sizes above one (the reference warns likewise).
    """

    def transport(payload: CompressedPayload, op: str) -> CompressedPayload:
        dist = _dist(import_module)
        dist.all_reduce(payload.buffer, op=_op(dist, op), **_group_kw(group))
        return payload

    return transport


def make_torch_async_all_reduce(*, group=None, import_module=_std_import):
    def transport(payload: CompressedPayload, op: str) -> HandleWork:
        dist = _dist(import_module)
        handle = dist.all_reduce(payload.buffer, op=_op(dist, op), async_op=True, **_group_kw(group))
        return HandleWork(handle, payload)

    return transport


def make_torch_tensor_all_reduce(*, group=None, import_module=_std_import) -> Callable[[Any, str], Any]:
    """Plain (uncompressed) in-place all-reduce; `mean` divides by the world size."""

    def transport(tensor: Any, op: str) -> Any:
        dist = _dist(import_module)
        kind = op.strip().lower()
        dist.all_reduce(tensor, op=_op(dist, "sum" if kind == "mean" else op), **_group_kw(group))
        if kind == "mean":
            tensor /= _world(dist, group)
        return tensor

    return transport


def _gather_buffers(dist, buffer, group, async_op: bool):
    world = _world(dist, group)
    slots = [buffer.new_empty(buffer.shape) for _ in range(world)]
    handle = dist.all_gather(slots, buffer, async_op=async_op, **_group_kw(group))
    return slots, handle


def make_torch_all_gather(*, group=None, import_module=_std_import) -> Callable[[Any], GatheredPayloads]:
    def transport(payload: Any) -> GatheredPayloads:
        dist = _dist(import_module)
        slots, _ = _gather_buffers(dist, payload_buffer(payload), group, False)
        return GatheredPayloads(tuple(slots))

    return transport


def make_torch_async_all_gather(*, group=None, import_module=_std_import) -> Callable[[Any], HandleWork]:
    def transport(payload: Any) -> HandleWork:
        dist = _dist(import_module)
        slots, handle = _gather_buffers(dist, payload_buffer(payload), group, True)
        return HandleWork(handle, GatheredPayloads(tuple(slots)))

    return transport


def make_torch_all_to_all(*, group=None, import_module=_std_import) -> Callable[[Sequence[Any]], list[Any]]:
    """Exchange one equally sized buffer with every rank; gloo lacks all_to_all, so
    there the exchange is emulated by one all_gather per source rank."""

    def transport(send: Sequence[Any]) -> list[Any]:
        dist = _dist(import_module)
        recv = [b.new_empty(b.shape) for b in send]
        try:
            dist.all_to_all(recv, list(send), **_group_kw(group))
            return recv
        except (RuntimeError, NotImplementedError):
            pass
        world = _world(dist, group)
        me = dist.get_rank(group) if group is not None else dist.get_rank()
        import torch

        stacked = torch.stack(list(send))
        everything = [stacked.new_empty(stacked.shape) for _ in range(world)]
        dist.all_gather(everything, stacked, **_group_kw(group))
        return [everything[src][me].clone() for src in range(world)]

    return transport
