"""Small value types passed between codecs and transports.

Parity: ccdl_comm/communication/collectives.py:10-41 and gather_reduce.py:10-45.
"""

from __future__ import annotations

from collections.abc import Callable, Mapping
from dataclasses import dataclass, field
from typing import Any

from ..config import CompressionConfig


@dataclass(frozen=True)
class CompressedPayload:
    buffer: Any
    shape: tuple[int, ...]
    dtype: str
    metadata: Mapping[str, Any] = field(default_factory=dict)

    def with_buffer(self, buffer: Any) -> "CompressedPayload":
        """Same shape, dtype and metadata around another buffer (what a transport returns after moving it)."""

        return CompressedPayload(buffer, self.shape, self.dtype, dict(self.metadata))


@dataclass(frozen=True)
class GatheredPayloads:
    """One payload per rank, in rank order.  `world_size` may be given, as transports written against the
    reference do (ccdl_comm/communication/gather_reduce.py:11-15); it defaults to the number of payloads
    and must agree with it."""

    payloads: tuple[Any, ...]
    world_size: int | None = None

    def __post_init__(self) -> None:
        payloads = tuple(self.payloads)
        object.__setattr__(self, "payloads", payloads)
        if self.world_size is None:
            object.__setattr__(self, "world_size", len(payloads))
        elif int(self.world_size) != len(payloads):
            raise ValueError(f"world_size {self.world_size} does not match {len(payloads)} gathered payloads")


def payload_buffer(payload: Any) -> Any:
    return payload.buffer if hasattr(payload, "buffer") else payload


def coerce_payload(value: Any, *, shape: tuple[int, ...], dtype: str) -> CompressedPayload:
    if isinstance(value, CompressedPayload):
        return value
    if isinstance(value, dict) and "buffer" in value:
        return CompressedPayload(value["buffer"], tuple(value.get("shape", shape)), str(value.get("dtype", dtype)),
                                 dict(value.get("metadata", {})))
    return CompressedPayload(value, shape, dtype)


@dataclass
class CompressedAllReduce:
    """compress -> all_reduce(payload) -> decompress (byte-sum transport, legacy)."""

    config: CompressionConfig
    compress: Callable[[Any, CompressionConfig], CompressedPayload]
    all_reduce: Callable[[CompressedPayload, str], CompressedPayload]
    decompress: Callable[[CompressedPayload, tuple[int, ...], CompressionConfig, str], Any]

    def run(self, tensor: Any, *, shape: tuple[int, ...], dtype: str, reduce: str = "mean") -> Any:
        reduced = self.all_reduce(self.compress(tensor, self.config), reduce)
        return self.decompress(reduced, shape, self.config, dtype)


@dataclass
class CompressedAllGatherReduce:
    """compress -> all_gather -> decompress each -> sum/mean (generic codec path)."""

    config: CompressionConfig
    compress: Callable[[Any, CompressionConfig], CompressedPayload]
    all_gather: Callable[[CompressedPayload], GatheredPayloads]
    decompress: Callable[[CompressedPayload, tuple[int, ...], CompressionConfig, str], Any]

    def run(self, tensor: Any, *, shape: tuple[int, ...], dtype: str, reduce: str = "mean") -> Any:
        if reduce not in ("mean", "sum"):
            raise ValueError(f"unsupported reduce {reduce!r}")
        gathered = self.all_gather(self.compress(tensor, self.config))
        parts = [self.decompress(p, shape, self.config, dtype) for p in gathered.payloads]
        if not parts:
            raise ValueError("all_gather returned no payloads")
        total = parts[0]
        for part in parts[1:]:
            total = total + part
        return total / len(parts) if reduce == "mean" else total
