"""Codec facade: the functions transports call to (de)quantize tensors.

Parity: ccdl_comm/quantization/codec.py:104-498 (same public names and
argument order).  CUDA tensors go to the sm_100a extension — the fused
`quant_push` / `reduce` kernels for the production profile (linear, top-k 0,
deterministic), the general kernels otherwise.  CPU tensors go to the bit-exact
torch oracle, which makes every transport testable without a GPU.  A CUDA
tensor without the extension is an error, never a silent fallback.
"""

from __future__ import annotations

from typing import Sequence

import torch

from ..config import CompressionConfig
from . import host_codec, oracle
from .loader import CudaExtensionStatus, require_extension
from .sizing import estimate_quantized_size

_DTYPE_CODE = {"fp16": 0, "bf16": 1, "fp32": 2}
_QUANT_CODE = {"linear": 0, "normal": 1, "uniform": 2, "e3m0": 3, "e2m1": 4}
MAX_FUSED_PAYLOADS = 16


def resolve_dtype(dtype: str, tensor: torch.Tensor | None = None) -> str:
    if dtype != "auto":
        if dtype not in _DTYPE_CODE:
            raise ValueError(f"unsupported dtype {dtype!r}")
        return dtype
    if tensor is None:
        raise ValueError("dtype='auto' needs a tensor to infer from")
    return oracle.dtype_name(tensor)


def is_fast_profile(config: CompressionConfig) -> bool:
    return config.quant_type == "linear" and config.topk == 0 and not config.stochastic


def _numel_of(shape) -> int:
    total = 1
    for dim in tuple(shape):
        total *= int(dim)
    return total


def _seed() -> int:
    return int(torch.randint(0, 2**62, (1,), dtype=torch.int64).item())


def allocate_quantized_buffer(tensor: torch.Tensor, config: CompressionConfig, *, dtype: str = "auto") -> torch.Tensor:
    name = resolve_dtype(dtype, tensor)
    size = estimate_quantized_size(tensor.numel(), dtype=name, config=config).quantized_bytes
    return torch.empty(size, dtype=torch.uint8, device=tensor.device)


def allocate_dequantized_buffer(tensor: torch.Tensor, shape, config: CompressionConfig) -> torch.Tensor:
    del config
    return torch.empty(tuple(shape), dtype=tensor.dtype, device=tensor.device)


# ---------------------------------------------------------------------------
# quantize
# ---------------------------------------------------------------------------
def _check_payload(buffer: torch.Tensor, numel: int, dtype: str, config: CompressionConfig) -> None:
    need = estimate_quantized_size(numel, dtype=dtype, config=config).quantized_bytes
    if buffer.dtype != torch.uint8:
        raise TypeError("payload must be a uint8 tensor")
    if buffer.numel() != need:
        raise ValueError(f"payload has {buffer.numel()} bytes, expected {need}")
    if not buffer.is_contiguous():
        raise ValueError("payload must be contiguous")


def _cuda_quantize(ext, flat: torch.Tensor, out: torch.Tensor, residual, prepared_out, config: CompressionConfig) -> None:
    groups = -(-flat.numel() // config.group_size)
    if is_fast_profile(config):
        mode = ext.PUSH_COMPACT_LOCAL if config.compact else ext.PUSH_BROADCAST
        ext.quant_push(flat, residual, prepared_out, None, [out.data_ptr()] if groups else [], mode,
                       0, groups, 0, config.group_size, config.bit, None, 0)
        return
    ext.quant_general(flat, residual, prepared_out, out, config.group_size, config.bit, config.topk,
                      _QUANT_CODE[config.quant_type], config.stochastic, config.compact,
                      _seed() if config.stochastic else 0)


def quantize_tensor(tensor: torch.Tensor, config: CompressionConfig, *,
                    extension_status: CudaExtensionStatus | None = None, output: torch.Tensor | None = None,
                    residual: torch.Tensor | None = None, metadata: dict | None = None,
                    prepared_out: torch.Tensor | None = None) -> torch.Tensor:
    """Quantize `tensor` (+ optional error-feedback `residual`) to a payload.

    `prepared_out` (an addition) receives T(tensor + residual); it may alias
    `residual`.  `metadata`, when a dict, is filled with the payload geometry.
    """

    name = oracle.dtype_name(tensor)
    flat = tensor.detach().reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    res = None if residual is None else residual.detach().reshape(-1)
    est = estimate_quantized_size(flat.numel(), dtype=name, config=config)
    if output is None:
        output = torch.empty(est.quantized_bytes, dtype=torch.uint8, device=tensor.device)
    else:
        _check_payload(output, flat.numel(), name, config)
    if metadata is not None:
        metadata.update(original_numel=flat.numel(), padded_numel=est.padded_numel, num_groups=est.num_groups,
                        dtype=name, compact=config.compact)
    if flat.numel() == 0:
        return output
    if tensor.is_cuda:
        ext = require_extension(extension_status)
        prep = None if prepared_out is None else prepared_out.detach().reshape(-1)
        _cuda_quantize(ext, flat, output, res, prep, config)
        return output
    prep = None if prepared_out is None else prepared_out.detach().reshape(-1)
    if (host_codec.serves(config) and output.is_contiguous() and (res is None or res.is_contiguous())
            and (prep is None or prep.is_contiguous())):
        host_codec.quantize(flat, config, name, output, res, prep)   # C++ twin of the oracle, bit-identical
        return output
    noise = None
    if config.stochastic:
        noise = torch.rand(est.padded_numel) - 0.5
    encoded = oracle.encode(flat, config, residual=res, noise=noise)
    output.copy_(encoded)
    if prepared_out is not None:
        prepared_out.reshape(-1).copy_(oracle.prepare(flat, res))
    return output


def inplace_quantize_pack(tensor: torch.Tensor, output: torch.Tensor, residual: torch.Tensor | None,
                          config: CompressionConfig, metadata: dict | None = None, *,
                          extension_status: CudaExtensionStatus | None = None) -> bool:
    """Fused residual-add + abs-max + quantize + pack into `output`.

    Returns False for profiles the fused kernel does not serve (the caller then
    uses `quantize_tensor`), mirroring codec.py:355-384 of the reference; unlike
    the reference both payload layouts are served.
    """

    if not is_fast_profile(config):
        return False
    quantize_tensor(tensor, config, extension_status=extension_status, output=output, residual=residual,
                    metadata=metadata)
    return True


# ---------------------------------------------------------------------------
# dequantize
# ---------------------------------------------------------------------------
def _prepare_output(output, shape, numel: int, torch_dtype, device) -> tuple[torch.Tensor, torch.Tensor]:
    if output is None:
        output = torch.empty(numel, dtype=torch_dtype, device=device)
    if output.numel() != numel:
        raise ValueError("output has the wrong number of elements")
    if output.dtype != torch_dtype:
        raise TypeError("output has the wrong dtype")
    if not output.is_contiguous():
        raise ValueError("output must be contiguous")
    return output, output.reshape(-1)


def dequantize_tensor(buffer: torch.Tensor, shape, config: CompressionConfig, *, dtype: str,
                      extension_status: CudaExtensionStatus | None = None, output: torch.Tensor | None = None,
                      reduce_op: str = "none") -> torch.Tensor:
    """Decode one payload; `reduce_op="sum"` adds into `output` in the source dtype."""

    if reduce_op not in ("none", "sum"):
        raise ValueError(f"unsupported reduce_op {reduce_op!r}")
    name = resolve_dtype(dtype)
    numel = _numel_of(shape)
    _check_payload(buffer, numel, name, config)
    if reduce_op == "sum" and output is None:
        raise ValueError("reduce_op='sum' needs an output to accumulate into")
    out, flat = _prepare_output(output, shape, numel, oracle.TORCH_DTYPES[name], buffer.device)
    if numel == 0:
        return out.reshape(tuple(shape))
    accumulate = reduce_op == "sum"
    if buffer.is_cuda:
        ext = require_extension(extension_status)
        groups = -(-numel // config.group_size)
        if is_fast_profile(config):
            ext.reduce([buffer.data_ptr()], groups, 0, config.compact, numel, _DTYPE_CODE[name], config.group_size,
                       config.bit, 1.0, flat, accumulate, None, None, [], 0, 0, None, None, 0)
        else:
            ext.dequant_general(buffer, flat, config.group_size, config.bit, config.topk,
                                _QUANT_CODE[config.quant_type], config.compact, accumulate)
    elif host_codec.serves(config) and flat.is_contiguous() and buffer.is_contiguous():
        host_codec.dequantize(buffer.reshape(-1), numel, config, name, flat, accumulate)
    elif accumulate:
        flat.copy_(oracle.decode_accumulate(buffer, flat, config))
    else:
        flat.copy_(oracle.decode(buffer, numel, config, name))
    return out.reshape(tuple(shape))


def _reduce_into(buffers: Sequence[torch.Tensor], flat_out: torch.Tensor, config: CompressionConfig, name: str,
                 divisor: float, extension_status, prepared=None, residual=None) -> None:
    """Shared body of the fused multi-payload reducers."""

    numel = flat_out.numel()
    for b in buffers:
        _check_payload(b, numel, name, config)
    if numel == 0:
        return
    if flat_out.is_cuda:
        ext = require_extension(extension_status)
        groups = -(-numel // config.group_size)
        if is_fast_profile(config) and len(buffers) <= MAX_FUSED_PAYLOADS:
            ext.reduce([b.data_ptr() for b in buffers], groups, 0, config.compact, numel, _DTYPE_CODE[name],
                       config.group_size, config.bit, 1.0 / divisor, flat_out, False,
                       None if prepared is None else prepared.reshape(-1),
                       None if residual is None else residual.reshape(-1), [], 0, 0, None, None, 0)
            return
        # general profiles: per-payload decode, accumulation in the source dtype
        for i, b in enumerate(buffers):
            if is_fast_profile(config):
                ext.reduce([b.data_ptr()], groups, 0, config.compact, numel, _DTYPE_CODE[name], config.group_size,
                           config.bit, 1.0, flat_out, i > 0, None, None, [], 0, 0, None, None, 0)
            else:
                ext.dequant_general(b, flat_out, config.group_size, config.bit, config.topk,
                                    _QUANT_CODE[config.quant_type], config.compact, i > 0)
        if divisor != 1.0:
            ext.scale_inplace(flat_out, 1.0 / divisor)
        if residual is not None:
            ext.error_feedback_update(prepared.reshape(-1), flat_out, residual.reshape(-1))
        return
    if is_fast_profile(config):
        prep_flat = None if prepared is None else prepared.reshape(-1)
        res_flat = None if residual is None else residual.reshape(-1)
        if (host_codec.serves(config) and flat_out.is_contiguous() and all(b.is_contiguous() for b in buffers)
                and (res_flat is None or (res_flat.is_contiguous() and prep_flat.is_contiguous()))):
            inv = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(divisor), dtype=torch.float32))
            host_codec.reduce([b.reshape(-1) for b in buffers], numel, config, name, inv, flat_out, prep_flat,
                              res_flat)
            return
        y, y32 = oracle.reduce_mean(buffers, numel, config, name, divisor)
        if residual is not None:
            residual.reshape(-1).copy_(oracle.residual_update(prepared, y32))
        flat_out.copy_(y)
        return
    acc = oracle.decode(buffers[0], numel, config, name)
    for b in buffers[1:]:
        acc = oracle.decode_accumulate(b, acc, config)
    if divisor != 1.0:
        acc = (acc.float() * (1.0 / divisor)).to(acc.dtype)
    if residual is not None:
        residual.reshape(-1).copy_(oracle.residual_update_from_restored(prepared, acc))
    flat_out.copy_(acc)


def _divisor(reduce: str, count: int) -> float:
    if reduce == "sum":
        return 1.0
    if reduce == "mean":
        return float(count)
    raise ValueError(f"unsupported reduce {reduce!r}; expected 'sum' or 'mean'")


def dequantize_reduce_tensors(buffers: Sequence[torch.Tensor], shape, config: CompressionConfig, *, dtype: str,
                              extension_status: CudaExtensionStatus | None = None,
                              output: torch.Tensor | None = None, reduce: str = "sum") -> torch.Tensor:
    if not buffers:
        raise ValueError("at least one payload is required")
    name = resolve_dtype(dtype)
    numel = _numel_of(shape)
    out, flat = _prepare_output(output, shape, numel, oracle.TORCH_DTYPES[name], buffers[0].device)
    _reduce_into(buffers, flat, config, name, _divisor(reduce, len(buffers)), extension_status)
    return out.reshape(tuple(shape))


def inplace_dequantize_reduce_mean(buffers: Sequence[torch.Tensor], output: torch.Tensor, config: CompressionConfig, *,
                                   extension_status: CudaExtensionStatus | None = None, reduce: str = "sum") -> bool:
    if not buffers or not is_fast_profile(config) or len(buffers) > MAX_FUSED_PAYLOADS:
        return False
    name = oracle.dtype_name(output)
    _reduce_into(buffers, output.reshape(-1), config, name, _divisor(reduce, len(buffers)), extension_status)
    return True


def inplace_dequantize_reduce_mean_update_error_feedback(
        buffers: Sequence[torch.Tensor], prepared: torch.Tensor, restored: torch.Tensor, residual: torch.Tensor,
        config: CompressionConfig, *, extension_status: CudaExtensionStatus | None = None,
        reduce: str = "sum") -> bool:
    """restored = reduce(buffers); residual = T(float(prepared) - restored_fp32), one kernel."""

    if not buffers or not is_fast_profile(config) or len(buffers) > MAX_FUSED_PAYLOADS:
        return False
    if not (prepared.numel() == restored.numel() == residual.numel()):
        raise ValueError("prepared, restored and residual must have the same number of elements")
    name = oracle.dtype_name(restored)
    _reduce_into(buffers, restored.reshape(-1), config, name, _divisor(reduce, len(buffers)), extension_status,
                 prepared=prepared, residual=residual)
    return True


def dequantize_reduce_update_error_feedback(buffers: Sequence[torch.Tensor], prepared: torch.Tensor,
                                            residual: torch.Tensor, shape, config: CompressionConfig, *, dtype: str,
                                            extension_status: CudaExtensionStatus | None = None,
                                            reduce: str = "sum") -> torch.Tensor:
    name = resolve_dtype(dtype)
    numel = _numel_of(shape)
    restored = torch.empty(numel, dtype=oracle.TORCH_DTYPES[name], device=buffers[0].device)
    _reduce_into(buffers, restored, config, name, _divisor(reduce, len(buffers)), extension_status,
                 prepared=prepared, residual=residual)
    return restored.reshape(tuple(shape))


def update_error_feedback_residual(prepared: torch.Tensor, restored: torch.Tensor, residual: torch.Tensor, *,
                                   extension_status: CudaExtensionStatus | None = None) -> torch.Tensor:
    """residual = T(float(prepared) - float(restored)), written in place."""

    if prepared.is_cuda:
        require_extension(extension_status).error_feedback_update(
            prepared.reshape(-1), restored.reshape(-1), residual.reshape(-1))
    else:
        residual.reshape(-1).copy_(oracle.residual_update_from_restored(prepared, restored))
    return residual
