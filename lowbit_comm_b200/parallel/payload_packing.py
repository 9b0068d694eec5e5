"""All-gather of payloads that carry tensor-valued metadata (e.g. fallback scales).

Parity: ccdl_comm/communication/payload_packing.py:14-160.  `make_payload_all_gather`
sends the buffer and each tensor metadata entry with separate collectives;
`FusedPayloadPacker` concatenates them into one byte tensor so a single
collective moves everything (worth it above ~4 M elements).
"""

from __future__ import annotations

from collections.abc import Callable, Mapping
from dataclasses import dataclass
from typing import Any

from .payload import CompressedPayload, GatheredPayloads, payload_buffer

DEFAULT_FUSED_PAYLOAD_MIN_NUMEL = 4_000_000


def _is_tensor(value: Any) -> bool:
    return hasattr(value, "dtype") and hasattr(value, "reshape") and hasattr(value, "numel")


def should_fuse_payload(tensor: Any, *, enabled: bool, min_numel: int = DEFAULT_FUSED_PAYLOAD_MIN_NUMEL) -> bool:
    if not enabled:
        return False
    count = tensor.numel() if callable(getattr(tensor, "numel", None)) else 0
    return count >= min_numel


def make_payload_all_gather(buffer_all_gather: Callable[[Any], GatheredPayloads]):
    """Gather `CompressedPayload`s: one collective for the buffer, one per tensor metadata entry."""

    def transport(payload: Any) -> GatheredPayloads:
        if not isinstance(payload, CompressedPayload):
            return buffer_all_gather(payload)
        buffers = buffer_all_gather(payload.buffer).payloads
        tensor_keys = [k for k, v in payload.metadata.items() if _is_tensor(v)]
        gathered_meta = {k: buffer_all_gather(payload.metadata[k]).payloads for k in tensor_keys}
        out = []
        for rank, buf in enumerate(buffers):
            meta = dict(payload.metadata)
            for k in tensor_keys:
                meta[k] = gathered_meta[k][rank]
            out.append(CompressedPayload(buf, payload.shape, payload.dtype, meta))
        return GatheredPayloads(tuple(out))

    return transport


@dataclass(frozen=True)
class TensorFieldSchema:
    """Where one tensor of a payload lives inside the packed byte tensor."""

    name: str
    dtype: Any
    shape: tuple[int, ...]
    numel: int
    byte_count: int
    offset: int


def _schema(name: str, tensor: Any, offset: int) -> TensorFieldSchema:
    return TensorFieldSchema(name, tensor.dtype, tuple(tensor.shape), int(tensor.numel()),
                             int(tensor.numel()) * int(tensor.element_size()), offset)


class FusedPayloadPacker:
    """Packs the buffer and the tensor-valued metadata of a payload into one uint8 tensor and back.

    The schema (names, dtypes, shapes, offsets) is fixed by the first payload (`from_payload`, or the first
    `pack` of an empty packer); every rank of an all-gather packs same-shaped payloads, so one schema
    decodes all of them.  Scalar metadata does not travel: it is copied from the schema's payload.
    """

    def __init__(self, buffer_schema: TensorFieldSchema | None = None,
                 metadata_schemas: tuple[TensorFieldSchema, ...] = (),
                 scalar_metadata: Mapping[str, Any] | None = None) -> None:
        self.buffer_schema = buffer_schema
        self.metadata_schemas = tuple(metadata_schemas)
        self.scalar_metadata = dict(scalar_metadata or {})

    @classmethod
    def from_payload(cls, payload: CompressedPayload) -> "FusedPayloadPacker":
        buffer_schema = _schema("buffer", payload.buffer, 0)
        cursor = buffer_schema.byte_count
        fields, scalars = [], {}
        for key, value in payload.metadata.items():
            if _is_tensor(value):
                fields.append(_schema(key, value, cursor))
                cursor += fields[-1].byte_count
            else:
                scalars[key] = value
        return cls(buffer_schema, tuple(fields), scalars)

    @property
    def packed_bytes(self) -> int:
        last = self.metadata_schemas[-1] if self.metadata_schemas else self.buffer_schema
        return 0 if last is None else last.offset + last.byte_count

    def _adopt(self, payload: CompressedPayload) -> None:
        made = FusedPayloadPacker.from_payload(payload)
        self.buffer_schema, self.metadata_schemas, self.scalar_metadata = \
            made.buffer_schema, made.metadata_schemas, made.scalar_metadata

    def pack(self, payload: CompressedPayload):
        import torch

        if self.buffer_schema is None:
            self._adopt(payload)
        parts = [(self.buffer_schema, payload.buffer)] + [(f, payload.metadata[f.name]) for f in self.metadata_schemas]
        for schema, tensor in parts:
            if tuple(tensor.shape) != schema.shape or tensor.dtype != schema.dtype:
                raise ValueError(f"payload field {schema.name!r} does not match the packer's schema")
        return torch.cat([t.contiguous().reshape(-1).view(torch.uint8) for _, t in parts])

    def unpack(self, packed, template: CompressedPayload | None = None, *, shape: tuple[int, ...] | None = None,
               dtype: str | None = None) -> CompressedPayload:
        """`unpack(packed, shape=..., dtype=...)` (the reference's form) or `unpack(packed, template)`."""

        if self.buffer_schema is None:
            raise RuntimeError("pack() or from_payload() must run before unpack()")
        if packed.numel() != self.packed_bytes:
            raise ValueError(f"packed payload has {packed.numel()} bytes, the schema describes {self.packed_bytes}")

        def piece(f: TensorFieldSchema):
            return packed[f.offset:f.offset + f.byte_count].view(f.dtype).reshape(f.shape)

        meta = dict(self.scalar_metadata if template is None else template.metadata)
        for f in self.metadata_schemas:
            meta[f.name] = piece(f)
        out_shape = tuple(shape) if shape is not None else (template.shape if template is not None else ())
        out_dtype = dtype if dtype is not None else (template.dtype if template is not None else "auto")
        return CompressedPayload(piece(self.buffer_schema), out_shape, out_dtype, meta)


@dataclass
class FusedPayloadAllGather:
    """Callable: packs, gathers the bytes with one collective, unpacks every rank's payload."""

    byte_all_gather: Callable[[Any], GatheredPayloads]
    packer: FusedPayloadPacker
    shape: tuple[int, ...]
    dtype: str

    def __call__(self, payload: CompressedPayload) -> GatheredPayloads:
        packed = self.packer.pack(payload)
        gathered = self.byte_all_gather(packed).payloads
        return GatheredPayloads(tuple(self.packer.unpack(p, shape=self.shape, dtype=self.dtype) for p in gathered))


def make_fused_payload_all_gather(buffer_all_gather: Callable[[Any], GatheredPayloads]):
    holder: dict[str, FusedPayloadAllGather] = {}

    def transport(payload: Any) -> GatheredPayloads:
        if not isinstance(payload, CompressedPayload):
            return buffer_all_gather(payload)
        if not any(_is_tensor(v) for v in payload.metadata.values()):
            got = buffer_all_gather(payload_buffer(payload)).payloads
            return GatheredPayloads(tuple(CompressedPayload(b, payload.shape, payload.dtype, dict(payload.metadata))
                                          for b in got))
        fused = holder.get("gather")
        if fused is None or fused.shape != tuple(payload.shape) or fused.dtype != payload.dtype \
                or fused.packer.buffer_schema.shape != tuple(payload.buffer.shape):
            fused = FusedPayloadAllGather(buffer_all_gather, FusedPayloadPacker.from_payload(payload),
                                          tuple(payload.shape), payload.dtype)
            holder["gather"] = fused
        return fused(payload)

    return transport
