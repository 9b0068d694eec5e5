"""All-reduce of integer codes under a shared scale: the library sums, nothing is decoded per payload.

Every group's scale is first agreed on (an all-reduce MAX over the ranks' abs-max values, 1/G of the data),
then every rank quantizes with that scale and the int8 codes are summed by the communication library itself
(`all_reduce` SUM on an int8 tensor, half the bytes of a bf16 all-reduce).  The reference offers this as its
explicit-only `overlap-scale` topology method and notes that it can overflow: W codes of up to 127 are added
in 8 bits (ccdl_comm/communication/topology_transport.py:716-748).  Here the codes are limited to
floor(127 / W) levels instead, so the sum always fits; the price is log2(W) bits of resolution, which is why
this stays an explicit choice (`make_native_topology_all_reduce(method="overlap-scale", hop_by_hop=True)`)
and is never picked automatically.  Plain torch operations: no kernels of this library are involved.
"""

from __future__ import annotations

from collections.abc import Callable
from importlib import import_module
from typing import Any

from ..config import CompressionConfig
from ..exceptions import UnsupportedCollective

CODE_LIMIT = 127


def shared_scale_levels(world_size: int) -> int:
    """Largest code magnitude a rank may use so that the sum over `world_size` ranks fits in int8."""

    if world_size <= 0:
        raise ValueError("world_size must be positive")
    levels = CODE_LIMIT // world_size
    if levels < 1:
        raise UnsupportedCollective(f"overlap-scale:W={world_size}", reason="more ranks than int8 code levels")
    return levels


def make_shared_scale_all_reduce(*, group: Any | None = None, dist: Any | None = None,
                                 torch: Any | None = None) -> Callable[..., Any]:
    """transport(tensor, *, config, op, async_op, dtype, extension_status=None) -> the reduced tensor (in
    place).  Only `config.group_size` is used; the wire carries one int8 code per element and one scale per
    group in the tensor's dtype (fp32 internally)."""

    def transport(tensor: Any, *, config: CompressionConfig, op: str = "mean", async_op: bool = False,
                  dtype: str = "auto", extension_status: Any | None = None) -> Any:
        if op not in ("sum", "mean"):
            raise UnsupportedCollective(f"overlap-scale:{op}", reason="only op='sum' and op='mean' are implemented")
        t = torch or import_module("torch")
        d = dist or import_module("torch.distributed")
        world = int(d.get_world_size(group))
        levels = shared_scale_levels(world)
        group_size = int(config.group_size)
        flat = tensor.reshape(-1)
        padded = -(-flat.numel() // group_size) * group_size
        values = t.zeros(padded, dtype=t.float32, device=tensor.device)
        values[: flat.numel()] = flat.float()
        grouped = values.reshape(-1, group_size)
        scale = grouped.abs().amax(dim=1, keepdim=True)
        d.all_reduce(scale, op=d.ReduceOp.MAX, group=group)
        step = t.clamp(scale, min=1.0e-6) / levels
        codes = t.clamp(t.round(grouped / step), -levels, levels).to(t.int8)
        d.all_reduce(codes, op=d.ReduceOp.SUM, group=group)
        if op == "mean":
            step = step / world
        flat.copy_((codes.float() * step).reshape(-1)[: flat.numel()].to(tensor.dtype))
        if async_op:
            from ..core.work import ImmediateWork

            return ImmediateWork(tensor)
        return tensor

    return transport
