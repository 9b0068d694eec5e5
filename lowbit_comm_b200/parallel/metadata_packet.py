"""Fixed-size metadata packet for dynamic-shape collectives.

Parity: ccdl_comm/cuda/metadata_packet.py:9-196 — protocol `tensor_v1`: sixteen
int64 words `[version, ndim, dtype_code, payload_numel, flags, 0, 0, 0, dims[8]]`
that travel through one `all_gather_into_tensor` instead of a pickled object
gather.  Pure Python; the torch side only views the words as an int64 tensor.
"""

from __future__ import annotations

from dataclasses import dataclass

PACKET_WORDS = 16
MAX_DIMS = 8
TENSOR_V1 = 1
DTYPE_CODES = {"fp16": 0, "bf16": 1, "fp32": 2}
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
