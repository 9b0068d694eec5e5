"""Wire-size contract of the low-bit payload.

Parity: ccdl_comm/quantization/sizing.py:36-91.  Per group the payload holds
`group_size*bit/8` value bytes plus metadata: the group scale stored in the
source dtype, and for top-k an index word and the k kept values, all in words
of the source element size (1, 3 or 4 words for topk 0/1/2).
"""

from __future__ import annotations

from dataclasses import dataclass

from ..config import CompressionConfig

DTYPE_BYTES = {"fp16": 2, "bf16": 2, "fp32": 4}
META_WORDS = {0: 1, 1: 3, 2: 4}


def dtype_bytes(dtype: str) -> int:
    if dtype not in DTYPE_BYTES:
        raise ValueError(f"Unsupported dtype={dtype!r}; expected one of {sorted(DTYPE_BYTES)}")
    return DTYPE_BYTES[dtype]


def value_bytes_per_group(config: CompressionConfig) -> int:
    return config.group_size * config.bit // 8


def metadata_bytes_per_group(dtype: str, topk: int) -> int:
    return META_WORDS[topk] * dtype_bytes(dtype)


def bytes_per_group(dtype: str, config: CompressionConfig) -> int:
    return value_bytes_per_group(config) + metadata_bytes_per_group(dtype, config.topk)


@dataclass(frozen=True)
class QuantizationSizeEstimate:
    numel: int
    padded_numel: int
    padding_numel: int
    num_groups: int
    original_bytes: int
    quantized_bytes: int
    compression_ratio: float


def estimate_quantized_size(numel: int, *, dtype: str, config: CompressionConfig) -> QuantizationSizeEstimate:
    """Bytes a tensor of `numel` elements occupies once quantized."""

    if numel < 0:
        raise ValueError("numel must be non-negative")
    width = dtype_bytes(dtype)
    groups = -(-numel // config.group_size)
    padded = groups * config.group_size
    packed = groups * bytes_per_group(dtype, config)
    raw = numel * width
    return QuantizationSizeEstimate(
        numel=numel, padded_numel=padded, padding_numel=padded - numel, num_groups=groups,
        original_bytes=raw, quantized_bytes=packed,
        compression_ratio=(raw / packed) if packed else 0.0)


@dataclass(frozen=True)
class WireLayout:
    """Byte offsets inside one payload (both layouts of the wire format).

    planar : [values of all groups][metadata of all groups]
    compact: per group [values][metadata], groups back to back
    (reference: csrc/quantization/quant_kernel.cuh:233-283 and 336-399).
    """

    num_groups: int
    value_bytes: int      # per group
    meta_bytes: int       # per group
    compact: bool

    @classmethod
    def of(cls, numel: int, dtype: str, config: CompressionConfig) -> "WireLayout":
        groups = -(-numel // config.group_size)
        return cls(groups, value_bytes_per_group(config), metadata_bytes_per_group(dtype, config.topk),
                   config.compact)

    @property
    def total_bytes(self) -> int:
        return self.num_groups * (self.value_bytes + self.meta_bytes)

    def value_offset(self, group: int) -> int:
        stride = self.value_bytes + (self.meta_bytes if self.compact else 0)
        return group * stride

    def meta_offset(self, group: int) -> int:
        if self.compact:
            return group * (self.value_bytes + self.meta_bytes) + self.value_bytes
        return self.num_groups * self.value_bytes + group * self.meta_bytes
