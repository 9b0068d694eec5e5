"""`compressed_all_gather` (parity: ccdl_comm/collectives/all_gather.py:24-68)."""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ...config import CompressionConfig
from ...core.work import CollectiveWork, ImmediateWork
from ...ops import codec
from ..payload import GatheredPayloads, coerce_payload, payload_buffer


def compressed_all_gather(
    tensor: Any,
    *,
    config: CompressionConfig,
    async_op: bool = False,
    dtype: str = "auto",
    quantize: Callable[[Any, CompressionConfig], Any] | None = None,
    dequantize: Callable[[Any, tuple[int, ...], CompressionConfig, str], Any] | None = None,
    all_gather: Callable[[Any], GatheredPayloads] | None = None,
    extension_status: Any | None = None,
    completion_manager: Any | None = None,
    group: Any | None = None,
) -> list[Any] | CollectiveWork[list[Any]]:
    """Every rank contributes a same-shaped tensor; returns the list of decoded tensors."""

    injected = any(v is not None for v in (quantize, dequantize, all_gather))
    if not injected:
        from ..communicator import get_communicator

        return get_communicator(group).all_gather(tensor, config=config, async_op=async_op, dtype=dtype)
    name = dtype if dtype != "auto" else codec.resolve_dtype(dtype, tensor)
    shape = tuple(tensor.shape)
    raw = quantize(tensor, config) if quantize is not None else codec.quantize_tensor(
        tensor, config, extension_status=extension_status)
    payload = coerce_payload(raw, shape=shape, dtype=name)
    if all_gather is None:
        from ..payload_packing import make_payload_all_gather
        from ..torch_transport import make_torch_all_gather

        all_gather = make_payload_all_gather(make_torch_all_gather(group=group))
    gathered = all_gather(payload)
    outs = []
    for p in gathered.payloads:
        if dequantize is not None:
            outs.append(dequantize(p, shape, config, name))
        else:
            outs.append(codec.dequantize_tensor(payload_buffer(p), shape, config, dtype=name,
                                                extension_status=extension_status))
    return ImmediateWork(outs) if async_op else outs
