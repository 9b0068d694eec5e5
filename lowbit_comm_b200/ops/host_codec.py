"""ctypes front end of the C++ host codec (`csrc/host_codec.cpp`, built as `_lbc_host.so`).

The CPU side of the codec facade uses it for every deterministic profile when
the library has been built (the fused multi-payload reduce for linear / top-k 0);
stochastic rounding, and a tree without the library, go through the torch oracle.  The two
are required to agree bit for bit (tests/test_host_codec.py), which makes this
an independent check of the oracle that the GPU kernels are tested against.
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

from ..config import CompressionConfig
from .sizing import estimate_quantized_size

_LIB_PATH = Path(__file__).resolve().parent / "_lbc_host.so"
_DTYPE_CODE = {"fp16": 0, "bf16": 1, "fp32": 2}
_TORCH = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_tried = False


def library() -> ctypes.CDLL | None:
    """The loaded host library, or None when it has not been built."""

    global _lib, _tried
    if _tried:
        return _lib
    with _lock:
        if _tried:
            return _lib
        if _LIB_PATH.exists():
            try:
                lib = ctypes.CDLL(str(_LIB_PATH))
                lib.lbc_host_abi_version.restype = ctypes.c_int
                if lib.lbc_host_abi_version() == 2:
                    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
                    lib.lbc_host_quantize.argtypes = [ci, ci, ci, ci, vp, vp, vp, i64, vp]
                    lib.lbc_host_dequantize.argtypes = [ci, ci, ci, ci, vp, i64, vp, ci]
                    lib.lbc_host_reduce.argtypes = [ci, ci, ci, ci, ctypes.POINTER(vp), ci, i64, ctypes.c_float, vp,
                                                    vp, vp]
                    lib.lbc_host_quantize_general.argtypes = [ci, ci, ci, ci, ci, ci, vp, vp, vp, i64, vp]
                    lib.lbc_host_dequantize_general.argtypes = [ci, ci, ci, ci, ci, ci, vp, i64, vp, ci]
                    for fn in (lib.lbc_host_quantize, lib.lbc_host_dequantize, lib.lbc_host_reduce,
                               lib.lbc_host_quantize_general, lib.lbc_host_dequantize_general):
                        fn.restype = ci
                    lib.lbc_host_half_to_float.argtypes, lib.lbc_host_half_to_float.restype = \
                        [ctypes.c_uint16], ctypes.c_float
                    lib.lbc_host_float_to_half.argtypes, lib.lbc_host_float_to_half.restype = \
                        [ctypes.c_float], ctypes.c_uint16
                    lib.lbc_host_float_to_bf16.argtypes, lib.lbc_host_float_to_bf16.restype = \
                        [ctypes.c_float], ctypes.c_uint16
                    _lib = lib
            except OSError:
                _lib = None
        _tried = True
    return _lib


_QUANT_CODE = {"linear": 0, "normal": 1, "uniform": 2, "e3m0": 3, "e2m1": 4}


def serves(config: CompressionConfig) -> bool:
    """Encode and decode: every deterministic profile (stochastic rounding stays with the torch oracle)."""

    return library() is not None and not config.stochastic and config.quant_type in _QUANT_CODE


def _fast(config: CompressionConfig) -> bool:
    return config.quant_type == "linear" and config.topk == 0


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, dtype: str, what: str) -> torch.Tensor:
    if t.device.type != "cpu" or t.dtype != _TORCH[dtype] or not t.is_contiguous():
        raise ValueError(f"{what} must be a contiguous CPU tensor of dtype {dtype}")
    return t


def quantize(x: torch.Tensor, config: CompressionConfig, dtype: str, out: torch.Tensor,
             residual: torch.Tensor | None = None, prepared_out: torch.Tensor | None = None) -> torch.Tensor:
    """Encode flat `x` (+ residual) into the uint8 payload `out`; `prepared_out` may alias `residual`."""

    lib = library()
    n = x.numel()
    need = estimate_quantized_size(n, dtype=dtype, config=config).quantized_bytes
    if out.dtype != torch.uint8 or out.numel() != need or not out.is_contiguous() or out.device.type != "cpu":
        raise ValueError(f"payload must be a contiguous CPU uint8 tensor of {need} bytes")
    for t, what in ((x, "input"), (residual, "residual"), (prepared_out, "prepared_out")):
        if t is not None:
            _check(t, dtype, what)
            if t.numel() != n:
                raise ValueError(f"{what} must have {n} elements")
    if _fast(config):
        rc = lib.lbc_host_quantize(_DTYPE_CODE[dtype], config.group_size, config.bit, int(config.compact), _ptr(x),
                                   _ptr(residual), _ptr(prepared_out), n, _ptr(out))
    else:
        rc = lib.lbc_host_quantize_general(_DTYPE_CODE[dtype], config.group_size, config.bit, config.topk,
                                           _QUANT_CODE[config.quant_type], int(config.compact), _ptr(x),
                                           _ptr(residual), _ptr(prepared_out), n, _ptr(out))
    if rc != 0:
        raise ValueError("host codec rejected the arguments")
    return out


def dequantize(payload: torch.Tensor, numel: int, config: CompressionConfig, dtype: str, out: torch.Tensor,
               accumulate: bool = False) -> torch.Tensor:
    lib = library()
    need = estimate_quantized_size(numel, dtype=dtype, config=config).quantized_bytes
    if payload.dtype != torch.uint8 or payload.numel() != need or not payload.is_contiguous():
        raise ValueError(f"payload has {payload.numel()} bytes, expected {need}")
    _check(out, dtype, "output")
    if out.numel() != numel:
        raise ValueError("output has the wrong number of elements")
    if _fast(config):
        rc = lib.lbc_host_dequantize(_DTYPE_CODE[dtype], config.group_size, config.bit, int(config.compact),
                                     _ptr(payload), numel, _ptr(out), int(accumulate))
    else:
        rc = lib.lbc_host_dequantize_general(_DTYPE_CODE[dtype], config.group_size, config.bit, config.topk,
                                             _QUANT_CODE[config.quant_type], int(config.compact), _ptr(payload),
                                             numel, _ptr(out), int(accumulate))
    if rc != 0:
        raise ValueError("host codec rejected the arguments")
    return out


def reduce(payloads: list[torch.Tensor], numel: int, config: CompressionConfig, dtype: str, scale: float,
           out: torch.Tensor | None, prepared: torch.Tensor | None = None,
           residual_out: torch.Tensor | None = None) -> None:
    """out = T(fp32 sum of the decoded payloads * scale); residual_out = T(float(prepared) - that fp32 value)."""

    if not _fast(config):
        raise ValueError("the fused host reduce serves linear / top-k 0 profiles")
    lib = library()
    need = estimate_quantized_size(numel, dtype=dtype, config=config).quantized_bytes
    for p in payloads:
        if p.dtype != torch.uint8 or p.numel() != need or not p.is_contiguous() or p.device.type != "cpu":
            raise ValueError(f"every payload must be a contiguous CPU uint8 tensor of {need} bytes")
    for t, what in ((out, "output"), (prepared, "prepared"), (residual_out, "residual_out")):
        if t is not None:
            _check(t, dtype, what)
            if t.numel() != numel:
                raise ValueError(f"{what} must have {numel} elements")
    array = (ctypes.c_void_p * len(payloads))(*[p.data_ptr() for p in payloads])
    rc = lib.lbc_host_reduce(_DTYPE_CODE[dtype], config.group_size, config.bit, int(config.compact), array,
                             len(payloads), numel, float(scale), _ptr(out), _ptr(prepared), _ptr(residual_out))
    if rc != 0:
        raise ValueError("host codec rejected the arguments")
