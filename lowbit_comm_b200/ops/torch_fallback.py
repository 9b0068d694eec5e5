"""Portable int8 codec made of stock torch ops (any device, any backend).

Parity: ccdl_comm/quantization/torch_fallback.py:10-53.  Not wire compatible
with the kernel payload on purpose: scales are fp32 `absmax/127` and travel as
a separate tensor in the payload metadata.  This is the codec of the CPU/gloo
DDP configuration.
"""

from __future__ import annotations

import torch

from ..config import CompressionConfig
from ..parallel.payload import CompressedPayload
from .oracle import TORCH_DTYPES, dtype_name


def quantize_tensor_fallback(tensor: torch.Tensor, config: CompressionConfig) -> CompressedPayload:
    if config.quant_type != "linear":
        raise ValueError("torch fallback supports only quant_type='linear'")
    if config.bit != 8:
        raise ValueError("torch fallback only supports bit=8")
    flat = tensor.reshape(-1)
    n = flat.numel()
    pad = (-n) % config.group_size
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    rows = flat.reshape(-1, config.group_size).float()
    scales = (rows.abs().amax(dim=1) / 127.0).clamp_min(torch.finfo(torch.float32).eps)
    codes = (rows / scales[:, None]).round_().clamp_(-127, 127).to(torch.int8)
    return CompressedPayload(buffer=codes.reshape(-1), shape=tuple(tensor.shape), dtype=dtype_name(tensor),
                             metadata={"scales": scales, "original_numel": n})


def dequantize_tensor_fallback(payload: CompressedPayload, shape, config: CompressionConfig, dtype: str) -> torch.Tensor:
    rows = payload.buffer.reshape(-1, config.group_size).float()
    scales = payload.metadata["scales"].reshape(-1, 1)
    n = int(payload.metadata["original_numel"])
    return (rows * scales).reshape(-1)[:n].to(TORCH_DTYPES[dtype]).reshape(tuple(shape))
