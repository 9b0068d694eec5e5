"""Fixed-size metadata packet for dynamic-shape collectives.

Parity: ccdl_comm/cuda/metadata_packet.py:9-196 — protocol `tensor_v1`: sixteen
int64 words `[version, ndim, dtype_code, payload_numel, flags, 0, 0, 0, dims[8]]`
that travel through one `all_gather_into_tensor` instead of a pickled object
gather.  Pure Python; the torch side only views the words as an int64 tensor.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from typing import Any

PACKET_WORDS = 16
MAX_DIMS = 8
TENSOR_V1 = 1
DTYPE_CODES = {"fp16": 1, "bf16": 2, "fp32": 3}   # the reference's codes (0 is never a valid dtype)
DTYPE_NAMES = {v: k for k, v in DTYPE_CODES.items()}
FLAG_EMPTY = 1


@dataclass(frozen=True)
class MetadataPacket:
    shape: tuple[int, ...]
    dtype: str
    payload_numel: int
    flags: int = 0
    version: int = TENSOR_V1

    def __post_init__(self) -> None:
        if len(self.shape) > MAX_DIMS:
            raise ValueError(f"at most {MAX_DIMS} dimensions fit a metadata packet")
        if any((not isinstance(d, int)) or d < 0 for d in self.shape):
            raise ValueError("dimensions must be non-negative integers")
        if self.dtype not in DTYPE_CODES:
            raise ValueError(f"unsupported dtype {self.dtype!r}")
        if self.payload_numel < 0:
            raise ValueError("payload_numel must be >= 0")

    @property
    def numel(self) -> int:
        total = 1
        for d in self.shape:
            total *= d
        return total

    def encode(self) -> list[int]:
        words = [self.version, len(self.shape), DTYPE_CODES[self.dtype], self.payload_numel, self.flags, 0, 0, 0]
        words += list(self.shape) + [0] * (MAX_DIMS - len(self.shape))
        return words

    @classmethod
    def decode(cls, words) -> "MetadataPacket":
        words = [int(w) for w in words]
        if len(words) != PACKET_WORDS:
            raise ValueError(f"a metadata packet has {PACKET_WORDS} words, got {len(words)}")
        version, ndim, code, payload, flags = words[:5]
        if version != TENSOR_V1:
            raise ValueError(f"unsupported metadata packet version {version}")
        if not 0 <= ndim <= MAX_DIMS:
            raise ValueError(f"invalid dimension count {ndim}")
        if code not in DTYPE_NAMES:
            raise ValueError(f"invalid dtype code {code}")
        if any(words[5:8]) or any(words[8 + ndim:]):
            raise ValueError("reserved words of the metadata packet must be zero")
        return cls(tuple(words[8:8 + ndim]), DTYPE_NAMES[code], payload, flags, version)


def decode_all(flat_words, world_size: int) -> list[MetadataPacket]:
    flat = [int(w) for w in flat_words]
    if len(flat) != world_size * PACKET_WORDS:
        raise ValueError("gathered metadata has the wrong length")
    return [MetadataPacket.decode(flat[r * PACKET_WORDS:(r + 1) * PACKET_WORDS]) for r in range(world_size)]


# ---- function-style interface with the reference's names ---------------------------------------
METADATA_PACKET_PROTOCOL_VERSION = TENSOR_V1
METADATA_PACKET_MAX_NDIM = MAX_DIMS
METADATA_PACKET_DIMS_OFFSET = 8
METADATA_PACKET_NUMEL = PACKET_WORDS
METADATA_PACKET_RESERVED_OFFSET = 5


def _check_packet_tensor(output: Any) -> None:
    count = output.numel() if callable(getattr(output, "numel", None)) else len(output)
    if count != PACKET_WORDS:
        raise ValueError(f"a metadata packet tensor holds {PACKET_WORDS} int64 words, got {count}")


def write_metadata_packet(output: Any, *, shape: Sequence[int], dtype: str, payload_numel: int, flags: int = 0) -> Any:
    """Overwrite an existing 16-word int64 tensor (or list) with the packet; no allocation."""

    for value, name in ((payload_numel, "payload_numel"), (flags, "flags")):
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError(f"{name} must be an integer")
        if value < 0:
            raise ValueError(f"{name} must be >= 0")
    if isinstance(shape, (str, bytes)) or not isinstance(shape, Sequence):
        raise TypeError("shape must be a sequence of integers")
    if any(isinstance(d, bool) or not isinstance(d, int) for d in shape):
        raise TypeError("shape must be a sequence of integers")
    _check_packet_tensor(output)
    words = MetadataPacket(tuple(shape), dtype, payload_numel, flags).encode()
    for index, word in enumerate(words):
        output[index] = word
    return output


def encode_metadata_packet(*, shape: Sequence[int], dtype: str, payload_numel: int, torch: Any, device: Any,
                           flags: int = 0, output: Any | None = None) -> Any:
    """The packet as an int64 tensor on `device` (`output`, when given, is overwritten and returned)."""

    packet = torch.empty(PACKET_WORDS, dtype=torch.int64, device=device) if output is None else output
    return write_metadata_packet(packet, shape=shape, dtype=dtype, payload_numel=payload_numel, flags=flags)


def _as_mapping(packet: MetadataPacket) -> Mapping[str, object]:
    return {"protocol_version": packet.version, "shape": packet.shape, "dtype": packet.dtype,
            "payload_numel": packet.payload_numel, "flags": packet.flags}


def decode_metadata_packet(packet: Any) -> Mapping[str, object]:
    """Validate one packet (one host read of a device tensor) and return its fields."""

    try:
        values = packet.tolist()
    except AttributeError as exc:
        raise RuntimeError("metadata packet must expose tolist()") from exc
    try:
        return _as_mapping(MetadataPacket.decode(values))
    except ValueError as exc:
        raise RuntimeError(str(exc)) from exc


def decode_metadata_packets(gathered_packet: Any, *, world_size: int) -> tuple[Mapping[str, object], ...]:
    """Decode a rank-major tensor of `world_size` packets with a single host read."""

    try:
        values = gathered_packet.tolist()
    except AttributeError as exc:
        raise RuntimeError("metadata packets must expose tolist()") from exc
    try:
        return tuple(_as_mapping(p) for p in decode_all(values, world_size))
    except ValueError as exc:
        raise RuntimeError(str(exc)) from exc
