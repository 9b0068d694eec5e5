"""All-gather of payloads that carry tensor-valued metadata (e.g. fallback scales).

Parity: ccdl_comm/communication/payload_packing.py:14-160.  `make_payload_all_gather`
sends the buffer and each tensor metadata entry with separate collectives;
`FusedPayloadPacker` concatenates them into one byte tensor so a single
collective moves everything (worth it above ~4 M elements).
"""

from __future__ import annotations

from collections.abc import Callable
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


class FusedPayloadPacker:
    """Packs buffer + tensor metadata into one uint8 tensor and back (schema cached)."""

    def __init__(self) -> None:
        self._schema: list[tuple[str, Any, tuple[int, ...], int]] | None = None

    def pack(self, payload: CompressedPayload):
        import torch

        parts = [("__buffer__", payload.buffer)] + [(k, v) for k, v in payload.metadata.items() if _is_tensor(v)]
        self._schema = [(k, v.dtype, tuple(v.shape), v.numel() * v.element_size()) for k, v in parts]
        return torch.cat([v.contiguous().reshape(-1).view(torch.uint8) for _, v in parts])

    def unpack(self, packed, template: CompressedPayload) -> CompressedPayload:
        if self._schema is None:
            raise RuntimeError("pack() must run before unpack()")
        meta = dict(template.metadata)
        cursor, buffer = 0, None
        for key, dtype, shape, nbytes in self._schema:
            piece = packed[cursor:cursor + nbytes].view(dtype).reshape(shape)
            cursor += nbytes
            if key == "__buffer__":
                buffer = piece
            else:
                meta[key] = piece
        return CompressedPayload(buffer, template.shape, template.dtype, meta)


def make_fused_payload_all_gather(buffer_all_gather: Callable[[Any], GatheredPayloads]):
    packer = FusedPayloadPacker()

    def transport(payload: Any) -> GatheredPayloads:
        if not isinstance(payload, CompressedPayload):
            return buffer_all_gather(payload)
        if not any(_is_tensor(v) for v in payload.metadata.values()):
            got = buffer_all_gather(payload_buffer(payload)).payloads
            return GatheredPayloads(tuple(CompressedPayload(b, payload.shape, payload.dtype, dict(payload.metadata))
                                          for b in got))
        packed = packer.pack(payload)
        return GatheredPayloads(tuple(packer.unpack(p, payload) for p in buffer_all_gather(packed).payloads))

    return transport
