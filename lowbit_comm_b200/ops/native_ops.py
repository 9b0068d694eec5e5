"""The reference's native op module, call for call, on top of this library's codec.

Code written against the reference sometimes skips its Python codec and calls the pybind module
`ccdl_cuda_ops` directly (ccdl_comm/csrc/pybind.cpp:133-166): positional arguments, enums instead of strings,
payload tensors in and out.  This module offers the same eleven functions, three enums and the ABI constant,
so that such code only has to change its import.  Nothing here has kernels of its own: every call builds the
`CompressionConfig` the arguments describe and goes through `ops.codec` -- the sm_100a kernels for CUDA
tensors, the C++ host codec or the oracle for CPU tensors -- so payloads are the same bytes either way.

Differences from the reference, all of them relaxations: inputs need not be padded to a multiple of the group
size; the functions that return `bool` ("did the fused kernel serve this?") return True for every 8- and 4-bit
linear profile in both layouts, not only for the compact one; CPU tensors are accepted.  `ReduceOP.MIN` and
`ReduceOP.MAX` exist in the enum, as in the reference, and are rejected, as they are there.
"""

from __future__ import annotations

import enum
from collections.abc import Sequence

import torch

from ..config import CompressionConfig
from . import codec, oracle, sizing

NATIVE_WORK_ABI_VERSION = 1


class ReduceOP(enum.Enum):
    SUM = 0
    MAX = 1
    MIN = 2
    NONE = 3


class QuantType(enum.Enum):
    Linear = 0
    Normal = 1
    Uniform = 2
    E3M0 = 3
    E2M1 = 4


class DType(enum.Enum):
    FP16 = 0
    BF16 = 1
    FP32 = 2


# pybind's `export_values()`: the members are also module attributes
SUM, MAX, MIN, NONE = ReduceOP.SUM, ReduceOP.MAX, ReduceOP.MIN, ReduceOP.NONE
Linear, Normal, Uniform, E3M0, E2M1 = QuantType
FP16, BF16, FP32 = DType

_DTYPE_NAME = {DType.FP16: "fp16", DType.BF16: "bf16", DType.FP32: "fp32"}
_REDUCE_NAME = {ReduceOP.NONE: "none", ReduceOP.SUM: "sum"}


def _config(group_size: int, topk: int, bit: int, quant_type: QuantType, compact: bool,
            stochastic: bool = False) -> CompressionConfig:
    return CompressionConfig(bit=int(bit), group_size=int(group_size), topk=int(topk),
                             quant_type=QuantType(quant_type).name.lower(), stochastic=bool(stochastic),
                             compact=bool(compact), allow_experimental=True, error_feedback=False)


def _reduce_name(reduce_op: ReduceOP) -> str:
    try:
        return _REDUCE_NAME[ReduceOP(reduce_op)]
    except KeyError:
        raise ValueError(f"dequantize supports ReduceOP.NONE and ReduceOP.SUM, not {reduce_op}") from None


def _decoded_numel(payload: torch.Tensor, dtype: str, config: CompressionConfig) -> int:
    """Elements a payload decodes to: whole groups, as in the reference (the caller trims the padding)."""

    if payload.dtype != torch.uint8:
        raise TypeError("input must be uint8")
    return payload.numel() // sizing.bytes_per_group(dtype, config) * config.group_size


# ---- quantize -------------------------------------------------------------------------------------------
def quantize(input: torch.Tensor, group_size: int, topk: int, stochastic: bool, bit: int,
             quant_type: QuantType = QuantType.Linear, compact: bool = False) -> torch.Tensor:
    return codec.quantize_tensor(input, _config(group_size, topk, bit, quant_type, compact, stochastic))


def inplace_quantize(input: torch.Tensor, output: torch.Tensor, group_size: int, topk: int, stochastic: bool,
                     bit: int, quant_type: QuantType = QuantType.Linear, compact: bool = False) -> None:
    codec.quantize_tensor(input, _config(group_size, topk, bit, quant_type, compact, stochastic), output=output)


def inplace_quantize_pack(input: torch.Tensor, output: torch.Tensor, residual: torch.Tensor | None, group_size: int,
                          topk: int, stochastic: bool, bit: int, quant_type: QuantType = QuantType.Linear,
                          compact: bool = True) -> bool:
    """Fused residual add + abs-max + quantize + pack of T(input + residual); `residual` is only read."""

    config = _config(group_size, topk, bit, quant_type, compact, stochastic)
    if not codec.is_fast_profile(config):
        return False
    codec.quantize_tensor(input, config, output=output, residual=residual)
    return True


# ---- dequantize -----------------------------------------------------------------------------------------
def inplace_dequantize(input: torch.Tensor, output: torch.Tensor, group_size: int, topk: int, bit: int,
                       reduce_op: ReduceOP = ReduceOP.NONE, quant_type: QuantType = QuantType.Linear,
                       compact: bool = False) -> None:
    codec.dequantize_tensor(input, tuple(output.shape), _config(group_size, topk, bit, quant_type, compact),
                            dtype=oracle.dtype_name(output), output=output, reduce_op=_reduce_name(reduce_op))


def dequantize(input: torch.Tensor, group_size: int, topk: int, bit: int, reduce_op: ReduceOP = ReduceOP.NONE,
               quant_type: QuantType = QuantType.Linear, dtype: DType = DType.FP16,
               compact: bool = False) -> torch.Tensor:
    _reduce_name(reduce_op)                      # a fresh output has nothing to add to: only validated
    config, name = _config(group_size, topk, bit, quant_type, compact), _DTYPE_NAME[DType(dtype)]
    return codec.dequantize_tensor(input, (_decoded_numel(input, name, config),), config, dtype=name)


def inplace_dequantize_reduce(inputs: Sequence[torch.Tensor], output: torch.Tensor, group_size: int, topk: int,
                              bit: int, quant_type: QuantType = QuantType.Linear, compact: bool = False) -> None:
    if not inputs:
        raise ValueError("inputs must not be empty")
    codec.dequantize_reduce_tensors(list(inputs), tuple(output.shape), _config(group_size, topk, bit, quant_type, compact),
                                    dtype=oracle.dtype_name(output), output=output, reduce="sum")


def dequantize_reduce(inputs: Sequence[torch.Tensor], group_size: int, topk: int, bit: int,
                      quant_type: QuantType = QuantType.Linear, dtype: DType = DType.FP16,
                      compact: bool = False) -> torch.Tensor:
    if not inputs:
        raise ValueError("inputs must not be empty")
    config, name = _config(group_size, topk, bit, quant_type, compact), _DTYPE_NAME[DType(dtype)]
    return codec.dequantize_reduce_tensors(list(inputs), (_decoded_numel(inputs[0], name, config),), config,
                                           dtype=name, reduce="sum")


def _fused_reduce(inputs, output, config: CompressionConfig, divisor: int, prepared=None, residual=None) -> bool:
    if divisor <= 0:
        raise ValueError("divisor must be > 0")
    if not inputs or not codec.is_fast_profile(config) or len(inputs) > codec.MAX_FUSED_PAYLOADS:
        return False
    codec._reduce_into(list(inputs), output.reshape(-1), config, oracle.dtype_name(output), float(divisor), None,
                       prepared=prepared, residual=residual)
    return True


def inplace_dequantize_reduce_mean(inputs: Sequence[torch.Tensor], output: torch.Tensor, group_size: int, topk: int,
                                   bit: int, quant_type: QuantType = QuantType.Linear, compact: bool = False,
                                   divisor: int = 1) -> bool:
    """output = T(sum of the decoded inputs / divisor), fp32 accumulation, one rounding."""

    return _fused_reduce(inputs, output, _config(group_size, topk, bit, quant_type, compact), divisor)


# ---- error feedback -------------------------------------------------------------------------------------
def inplace_error_feedback_update(prepared: torch.Tensor, restored: torch.Tensor, residual: torch.Tensor) -> None:
    codec.update_error_feedback_residual(prepared, restored, residual)


def inplace_dequantize_reduce_mean_update_error_feedback(
        inputs: Sequence[torch.Tensor], prepared: torch.Tensor, restored: torch.Tensor, residual: torch.Tensor,
        group_size: int, topk: int, bit: int, quant_type: QuantType = QuantType.Linear, compact: bool = False,
        divisor: int = 1) -> bool:
    """restored as in `inplace_dequantize_reduce_mean`; residual = T(float(prepared) - the fp32 mean)."""

    if not (prepared.numel() == restored.numel() == residual.numel()):
        raise ValueError("prepared, restored and residual must have the same number of elements")
    return _fused_reduce(inputs, restored, _config(group_size, topk, bit, quant_type, compact), divisor,
                         prepared=prepared, residual=residual)


def dequantize_reduce_update_error_feedback(
        inputs: Sequence[torch.Tensor], prepared: torch.Tensor, residual: torch.Tensor, group_size: int, topk: int,
        bit: int, quant_type: QuantType = QuantType.Linear, dtype: DType = DType.FP16, compact: bool = False,
        divisor: int = 1) -> torch.Tensor:
    """Allocating form: returns `restored`; profiles the fused kernel does not serve are decoded payload by
    payload, divided, and the residual is updated from the rounded result."""

    if not inputs:
        raise ValueError("inputs must not be empty")
    if divisor <= 0:
        raise ValueError("divisor must be > 0")
    config, name = _config(group_size, topk, bit, quant_type, compact), _DTYPE_NAME[DType(dtype)]
    restored = torch.empty(_decoded_numel(inputs[0], name, config), dtype=oracle.TORCH_DTYPES[name],
                           device=inputs[0].device)
    if restored.numel() != prepared.numel():
        raise ValueError("prepared must have as many elements as the payloads decode to")
    codec._reduce_into(list(inputs), restored, config, name, float(divisor), None, prepared=prepared,
                       residual=residual)
    return restored
