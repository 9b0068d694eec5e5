"""Bit-exact reference codec for the wire format, written with plain torch ops.

This file is the numerical specification every sm_100a kernel is tested
against; it runs on CPU.  It restates the math of the reference's CUDA kernels
(csrc/quantization/quant_pack_kernel.cu:25-163, quant_kernel.cuh:25-153,
dequant_kernel.cuh:15-44, dequant_reduce_kernel.cu:38-221, inner.cuh:9-96):

* prepared = T(float(x) + float(residual))            (rounded to T first)
* stored scale s = T(max |prepared|) per group; with top-k the k largest
  magnitudes are pulled out (kept verbatim) and s is the (k+1)-th largest
* linear: q = clamp(rint(float(p) * (L / max(float(s), 1e-6))), -L, L), L=127|7
* code-book (4-bit): index of the nearest entry of a 15-entry table of p/s
* words are as wide as T and hold their elements most-significant first
* decode: x^ = T(float(q) * (float(s) / L))   or   T(table[q] * float(s))
* fused mean: y = T((sum_r x^_r in fp32) * (1/W)); residual' = T(float(p) - y32)

Top-k tie-breaking (equal magnitudes) is first-occurrence for 16-bit sources
and last-occurrence for fp32 sources; a decoder never depends on it.
"""

from __future__ import annotations

import torch

from ..config import CompressionConfig
from .sizing import META_WORDS, WireLayout

TORCH_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
NAME_OF = {v: k for k, v in TORCH_DTYPES.items()}
_INT_VIEW = {2: torch.int16, 4: torch.int32}

_INF = float("inf")
CODEBOOKS = {
    "normal": [-1.0, -0.815410147, -0.655160150, -0.510228027, -0.375324982, -0.246951370, -0.122538030, 0.0,
               0.122538030, 0.246951370, 0.375324982, 0.510228027, 0.655160150, 0.815410147, 1.0, _INF],
    "uniform": [-1.0, -0.85714286, -0.71428571, -0.57142857, -0.42857143, -0.28571429, -0.14285714, 0.0,
                0.14285714, 0.28571429, 0.42857143, 0.57142857, 0.71428571, 0.85714286, 1.0, _INF],
    "e3m0": [-1.0, -0.5, -0.25, -0.125, -0.0625, -0.03125, -0.015625, 0.0,
             0.015625, 0.03125, 0.0625, 0.125, 0.25, 0.5, 1.0, _INF],
    "e2m1": [-1.0, -0.6666666666666666, -0.5, -0.3333333333333333, -0.25, -0.16666666666666666, -0.125, 0.0,
             0.125, 0.16666666666666666, 0.25, 0.3333333333333333, 0.5, 0.6666666666666666, 1.0, _INF],
}


def dtype_name(tensor_or_dtype) -> str:
    dt = tensor_or_dtype.dtype if isinstance(tensor_or_dtype, torch.Tensor) else tensor_or_dtype
    if dt not in NAME_OF:
        raise ValueError(f"unsupported source dtype {dt}")
    return NAME_OF[dt]


def codebook(name: str) -> torch.Tensor:
    return torch.tensor(CODEBOOKS[name], dtype=torch.float32)


def _levels(bit: int) -> float:
    return 127.0 if bit == 8 else 7.0


def prepare(x: torch.Tensor, residual: torch.Tensor | None) -> torch.Tensor:
    """Error-feedback compensation, rounded to the source dtype."""

    flat = x.reshape(-1)
    if residual is None:
        return flat
    return (flat.float() + residual.reshape(-1).float()).to(x.dtype)


def _grouped(flat: torch.Tensor, group: int) -> torch.Tensor:
    pad = (-flat.numel()) % group
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    return flat.reshape(-1, group)


def _pull_topk(groups: torch.Tensor, k: int, last_wins: bool):
    """Remove the k largest magnitudes per group; returns (rest, idx[k], val[k])."""

    rest = groups.clone()
    mag = rest.float().abs()
    g = rest.shape[1]
    idxs, vals = [], []
    taken = torch.zeros_like(mag, dtype=torch.bool)
    for _ in range(k):
        cand = mag.masked_fill(taken, -1.0)
        if last_wins:
            pos = g - 1 - torch.argmax(cand.flip(1), dim=1)
        else:
            pos = torch.argmax(cand, dim=1)
        idxs.append(pos)
        vals.append(rest.gather(1, pos[:, None])[:, 0].clone())
        taken.scatter_(1, pos[:, None], True)
    rest = rest.masked_fill(taken, 0)
    return rest, idxs, vals


def _pack_words(codes: torch.Tensor, bit: int, word_bytes: int) -> torch.Tensor:
    """codes: int64 [groups, G] of unsigned fields -> uint8 [groups, G*bit/8]."""

    if bit == 8:
        by = codes.to(torch.uint8)
    else:
        by = ((codes[:, 0::2] << 4) | codes[:, 1::2]).to(torch.uint8)
    groups = by.shape[0]
    return by.reshape(groups, -1, word_bytes).flip(2).reshape(groups, -1).contiguous()


def _unpack_words(raw: torch.Tensor, bit: int, word_bytes: int) -> torch.Tensor:
    """uint8 [groups, G*bit/8] -> int64 [groups, G] unsigned fields."""

    groups = raw.shape[0]
    by = raw.reshape(groups, -1, word_bytes).flip(2).reshape(groups, -1).to(torch.int64)
    if bit == 8:
        return by
    return torch.stack([by >> 4, by & 15], dim=2).reshape(groups, -1)


def encode(x: torch.Tensor, config: CompressionConfig, residual: torch.Tensor | None = None,
           noise: torch.Tensor | None = None) -> torch.Tensor:
    """Quantize `x` (any shape) to a uint8 payload in the wire format.

    `noise`, when given, holds the stochastic-rounding offsets (uniform in
    (-0.5, 0.5]) per padded element; without it rounding is to nearest even.
    """

    name = dtype_name(x)
    word = x.element_size()
    p = prepare(x.detach().cpu(), None if residual is None else residual.detach().cpu())
    groups = _grouped(p, config.group_size)
    n_groups = groups.shape[0]
    if n_groups == 0:
        return torch.empty(0, dtype=torch.uint8)
    rest, idxs, vals = (groups, [], [])
    if config.topk:
        rest, idxs, vals = _pull_topk(groups, config.topk, last_wins=(name == "fp32"))
    stored = rest.float().abs().amax(dim=1).to(x.dtype)            # scale in source dtype
    safe = stored.float().clamp_min(1e-6)
    values = rest.float()
    if config.quant_type == "linear":
        lim = _levels(config.bit)
        mul = (torch.tensor(lim, dtype=torch.float32) / safe)[:, None]
        t = values * mul
        if noise is not None:
            t = t + noise.reshape(n_groups, -1).float()
        q = torch.round(t).clamp_(-lim, lim).to(torch.int64)
        codes = q & (255 if config.bit == 8 else 15)
    else:
        if config.bit != 4:
            raise ValueError("code-book quantization is 4-bit only")
        table = codebook(config.quant_type)
        t = values / safe[:, None]
        low = (torch.searchsorted(table[:15].contiguous(), t.contiguous(), right=True) - 1).clamp_(0, 14)
        gap = table[low + 1] - table[low]
        if noise is not None:
            up = (noise.reshape(n_groups, -1).float() + 0.5) < (t - table[low]) / gap
        else:
            up = (t - table[low]) > gap / 2
        codes = (low + up.to(torch.int64)).to(torch.int64)
    value_bytes = _pack_words(codes, config.bit, word)

    iview = _INT_VIEW[word]
    meta = torch.zeros(n_groups, META_WORDS[config.topk], dtype=iview)
    meta[:, 0] = stored.view(iview)
    if config.topk >= 1:
        index_word = idxs[0].clone()
        if config.topk == 2:
            index_word = index_word | (idxs[1] << 8)
        meta[:, 1] = index_word.to(iview)
        meta[:, 2] = vals[0].view(iview)
        if config.topk == 2:
            meta[:, 3] = vals[1].view(iview)
    meta_bytes = meta.view(torch.uint8).reshape(n_groups, -1)
    if config.compact:
        return torch.cat([value_bytes, meta_bytes], dim=1).reshape(-1).contiguous()
    return torch.cat([value_bytes.reshape(-1), meta_bytes.reshape(-1)]).contiguous()


def _split(payload: torch.Tensor, numel: int, config: CompressionConfig, dtype: str):
    layout = WireLayout.of(numel, dtype, config)
    raw = payload.detach().cpu().reshape(-1)
    if raw.numel() != layout.total_bytes:
        raise ValueError(f"payload has {raw.numel()} bytes, expected {layout.total_bytes}")
    g = layout.num_groups
    if config.compact:
        rec = raw.reshape(g, layout.value_bytes + layout.meta_bytes)
        return rec[:, :layout.value_bytes].contiguous(), rec[:, layout.value_bytes:].contiguous()
    split = g * layout.value_bytes
    return raw[:split].reshape(g, layout.value_bytes), raw[split:].reshape(g, layout.meta_bytes)


def decode_fp32(payload: torch.Tensor, numel: int, config: CompressionConfig, dtype: str) -> torch.Tensor:
    """Dequantize to fp32 *before* the final rounding to the source dtype.

    Top-k values are exact source-dtype values, so they are already rounded.
    """

    tdt = TORCH_DTYPES[dtype]
    word = 2 if dtype != "fp32" else 4
    if numel == 0:
        return torch.empty(0, dtype=torch.float32)
    vbytes, mbytes = _split(payload, numel, config, dtype)
    iview = _INT_VIEW[word]
    meta = mbytes.contiguous().view(iview).reshape(vbytes.shape[0], -1)
    scale = meta[:, 0].contiguous().view(tdt).float()
    codes = _unpack_words(vbytes, config.bit, word)
    if config.quant_type == "linear":
        lim = _levels(config.bit)
        half = 128 if config.bit == 8 else 8
        signed = torch.where(codes >= half, codes - 2 * half, codes).float()
        out = signed * (scale / torch.tensor(lim, dtype=torch.float32))[:, None]
    else:
        out = codebook(config.quant_type)[codes] * scale[:, None]
    if config.topk:
        index_word = meta[:, 1].to(torch.int64) & 0xFFFF
        out = out.to(tdt).float()  # the non-top-k values are rounded before top-k is written back
        for j in range(config.topk):
            pos = (index_word >> (8 * j)) & 0xFF
            val = meta[:, 2 + j].contiguous().view(tdt).float()
            out.scatter_(1, pos[:, None], val[:, None])
    return out.reshape(-1)[:numel]


def _codes_and_steps(payload: torch.Tensor, numel: int, config: CompressionConfig, dtype: str):
    """Linear profiles: signed integer codes and the per-element step `scale / L`, both fp32."""

    tdt = TORCH_DTYPES[dtype]
    word = 2 if dtype != "fp32" else 4
    vbytes, mbytes = _split(payload, numel, config, dtype)
    meta = mbytes.contiguous().view(_INT_VIEW[word]).reshape(vbytes.shape[0], -1)
    scale = meta[:, 0].contiguous().view(tdt).float()
    codes = _unpack_words(vbytes, config.bit, word)
    half = 128 if config.bit == 8 else 8
    signed = torch.where(codes >= half, codes - 2 * half, codes).float()
    step = (scale / torch.tensor(_levels(config.bit), dtype=torch.float32))[:, None].expand_as(signed)
    return signed.reshape(-1)[:numel], step.reshape(-1)[:numel]


def local_error(prepared: torch.Tensor, payload: torch.Tensor, config: CompressionConfig) -> torch.Tensor:
    """This rank's own quantization error T(prepared - code * step), one fused rounding."""

    name = dtype_name(prepared)
    code, step = _codes_and_steps(payload, prepared.numel(), config, name)
    err = (prepared.reshape(-1).double() - code.double() * step.double()).float()
    return err.to(prepared.dtype)


def decode(payload: torch.Tensor, numel: int, config: CompressionConfig, dtype: str) -> torch.Tensor:
    return decode_fp32(payload, numel, config, dtype).to(TORCH_DTYPES[dtype])


def decode_accumulate(payload: torch.Tensor, into: torch.Tensor, config: CompressionConfig) -> torch.Tensor:
    """Unfused SUM path: `into += decode(payload)` in the source dtype."""

    name = dtype_name(into)
    add = decode(payload, into.numel(), config, name).reshape(into.shape)
    return (into.float() + add.float()).to(into.dtype)


def reduce_mean(payloads, numel: int, config: CompressionConfig, dtype: str, divisor: float | None = None):
    """Fused multi-payload reduce: fp32 accumulate in payload order, one rounding.

    Returns (T result, fp32 result).  `divisor=None` means the payload count.
    """

    acc = torch.zeros(numel, dtype=torch.float32)
    fused = config.quant_type == "linear" and config.topk == 0
    for p in payloads:
        if fused:
            # the kernels accumulate with one fused multiply-add per payload:
            # acc = round_fp32(code * step + acc), emulated here in float64
            code, step = _codes_and_steps(p, numel, config, dtype)
            acc = (code.double() * step.double() + acc.double()).float()
        else:
            acc = acc + decode_fp32(p, numel, config, dtype)
    div = float(len(payloads)) if divisor is None else float(divisor)
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(div, dtype=torch.float32)
    y32 = acc * inv
    return y32.to(TORCH_DTYPES[dtype]), y32


def residual_update(prepared: torch.Tensor, reduced_fp32: torch.Tensor) -> torch.Tensor:
    """Reference error-feedback rule: residual' = T(float(prepared) - mean_fp32)."""

    return (prepared.reshape(-1).float() - reduced_fp32.reshape(-1)).to(prepared.dtype)


def residual_update_from_restored(prepared: torch.Tensor, restored: torch.Tensor) -> torch.Tensor:
    """Unfused rule: residual' = T(float(prepared) - float(restored))."""

    return (prepared.reshape(-1).float() - restored.reshape(-1).float()).to(prepared.dtype)
