"""`Quantizer`: one compression profile and one element type bound to the codec.

For code that encodes and decodes many tensors with the same settings (a gradient hook, a checkpoint
compressor, a notebook).  It adds nothing to the math -- `ops.codec` does the work, on the GPU through the
sm_100a kernels and on the CPU through the host codec -- but it remembers the profile, answers size questions
without touching a tensor, and can measure what a round trip costs in accuracy.  Method names follow the
reference's facade (ccdl_comm/quantization/quantizer.py:10-67); `roundtrip`, `error`, `wire_bytes` and the
`residual=` argument are additions.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch

from ..config import CompressionConfig
from . import codec, sizing
from .loader import CudaExtensionStatus


class _IsQuantized:
    """`Quantizer.is_quantized(value)`: does `value` look like a payload (uint8 tensor)?
    `quantizer.is_quantized()`: does this profile compress at all (fewer than 16 bits per element)?"""

    @staticmethod
    def _holds_codes(value: Any) -> bool:
        return isinstance(value, torch.Tensor) and value.dtype == torch.uint8

    def __get__(self, instance: "Quantizer | None", owner: type) -> Callable[..., bool]:
        if instance is None:
            return self._holds_codes

        def answer(*value: Any) -> bool:
            return self._holds_codes(value[0]) if value else instance.config.bit < 16

        return answer


class Quantizer:
    is_quantized = _IsQuantized()

    def __init__(self, config: CompressionConfig | None = None, *, dtype: str = "auto",
                 extension_status: CudaExtensionStatus | None = None,
                 quantize_fn: Callable[..., Any] | None = None, dequantize_fn: Callable[..., Any] | None = None,
                 allocate_fn: Callable[..., Any] | None = None) -> None:
        self.config = CompressionConfig() if config is None else config
        self.dtype = dtype
        self.extension_status = extension_status
        # the three codec entry points can be replaced (tests, a recording shim, another device's codec)
        self._encode = quantize_fn or codec.quantize_tensor
        self._decode = dequantize_fn or codec.dequantize_tensor
        self._allocate = allocate_fn or codec.allocate_quantized_buffer

    # -- the element type ---------------------------------------------------------------------------
    def _dtype_for(self, override: str | None, tensor: torch.Tensor | None = None) -> str:
        name = override or self.dtype
        if name != "auto":
            return name
        if tensor is None:
            raise ValueError("dequantize needs an explicit dtype ('fp16', 'bf16' or 'fp32')")
        return codec.resolve_dtype(name, tensor)

    # -- encode / decode ----------------------------------------------------------------------------
    def quantize(self, tensor: torch.Tensor, output: torch.Tensor | None = None, *,
                 residual: torch.Tensor | None = None) -> torch.Tensor:
        extra = {} if residual is None else {"residual": residual}
        return self._encode(tensor, self.config, extension_status=self.extension_status, output=output, **extra)

    def dequantize(self, buffer: torch.Tensor, shape, output: torch.Tensor | None = None, *,
                   reduce_op: str = "none", dtype: str | None = None) -> torch.Tensor:
        return self._decode(buffer, shape, self.config, dtype=self._dtype_for(dtype),
                            extension_status=self.extension_status, output=output, reduce_op=reduce_op)

    def roundtrip(self, tensor: torch.Tensor) -> torch.Tensor:
        """What a receiver would see: decode(encode(tensor)), same shape and dtype as `tensor`."""

        return self.dequantize(self.quantize(tensor), tuple(tensor.shape), dtype=self._dtype_for(None, tensor))

    def error(self, tensor: torch.Tensor) -> dict[str, float]:
        """Accuracy of one round trip, in fp32: largest and rms absolute error, and rms error relative to
        the rms of the input."""

        exact = tensor.detach().float()
        delta = self.roundtrip(tensor).float() - exact
        rms = delta.pow(2).mean().sqrt().item() if delta.numel() else 0.0
        scale = exact.pow(2).mean().sqrt().item() if exact.numel() else 0.0
        return {"max_abs": delta.abs().max().item() if delta.numel() else 0.0, "rms": rms,
                "relative_rms": rms / scale if scale > 0 else 0.0}

    # -- sizes --------------------------------------------------------------------------------------
    def allocate_q(self, tensor: torch.Tensor, *, dtype: str | None = None) -> torch.Tensor:
        return self._allocate(tensor, self.config, dtype=dtype or self.dtype)

    def wire_bytes(self, numel: int, *, dtype: str | None = None) -> int:
        return sizing.estimate_quantized_size(numel, dtype=self._dtype_for(dtype), config=self.config).quantized_bytes

    # -- persistence --------------------------------------------------------------------------------
    def to_dict(self) -> dict:
        return {"config": self.config.to_dict(), "dtype": self.dtype}

    @classmethod
    def from_dict(cls, data: dict, **kwargs) -> "Quantizer":
        return cls(CompressionConfig.from_dict(data.get("config", {})), dtype=str(data.get("dtype", "auto")), **kwargs)

    def __repr__(self) -> str:
        return f"Quantizer(bit={self.config.bit}, group_size={self.config.group_size}, dtype={self.dtype!r})"
