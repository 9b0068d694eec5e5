"""Object-style facade over the codec (parity: ccdl_comm/quantization/quantizer.py:10-67)."""

from __future__ import annotations

import torch

from ..config import CompressionConfig
from . import codec
from .loader import CudaExtensionStatus


class Quantizer:
    def __init__(self, config: CompressionConfig | None = None, *, dtype: str = "auto",
                 extension_status: CudaExtensionStatus | None = None) -> None:
        self.config = config or CompressionConfig()
        self.dtype = dtype
        self._status = extension_status

    def quantize(self, tensor: torch.Tensor, *, output: torch.Tensor | None = None,
                 residual: torch.Tensor | None = None) -> torch.Tensor:
        return codec.quantize_tensor(tensor, self.config, extension_status=self._status, output=output,
                                     residual=residual)

    def dequantize(self, buffer: torch.Tensor, shape, *, dtype: str | None = None,
                   output: torch.Tensor | None = None, reduce_op: str = "none") -> torch.Tensor:
        name = dtype or self.dtype
        if name == "auto":
            raise ValueError("dequantize needs an explicit dtype ('fp16', 'bf16' or 'fp32')")
        return codec.dequantize_tensor(buffer, shape, self.config, dtype=name, extension_status=self._status,
                                       output=output, reduce_op=reduce_op)

    def allocate_q(self, tensor: torch.Tensor) -> torch.Tensor:
        return codec.allocate_quantized_buffer(tensor, self.config, dtype=self.dtype)

    @staticmethod
    def is_quantized(value) -> bool:
        return isinstance(value, torch.Tensor) and value.dtype == torch.uint8

    def to_dict(self) -> dict:
        return {"config": self.config.to_dict(), "dtype": self.dtype}

    @classmethod
    def from_dict(cls, data: dict, **kwargs) -> "Quantizer":
        return cls(CompressionConfig.from_dict(data.get("config", {})), dtype=data.get("dtype", "auto"), **kwargs)
