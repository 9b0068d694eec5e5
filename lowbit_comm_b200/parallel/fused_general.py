"""Compressed all-reduce over peer memory for the profiles the production kernels do not serve:
top-k outliers (1 or 2 values per group kept verbatim), the 4-bit code-books, stochastic rounding.

The reference sends any `CompressionConfig` through every collective because its transports call the one
codec and move the payload with NCCL (ccdl_comm/quantization/codec.py:104-158, top-k selection
csrc/quantization/quant_kernel.cuh:38-97, records :249-257, write-back dequant_kernel.cuh:130-148).  Here
such a profile takes two kernels that fuse the codec with the movement; no NCCL call is involved:

  quant_general (push)  x (+ residual) -> payload (values, scale, top-k index word and values), every
                        piece stored straight into slot [me] of every rank's receive region (own memory and
                        peer stores over NVLink); `prepared` parked in the residual buffer; the last block
                        of the grid raises a release signal on every rank
  reduce_general        bounded wait for the W signals, then ONE pass: decode every slot, accumulate in the
                        source dtype in rank order (the reference's unfused SUM rule), scale by 1/W for a
                        mean, write the result and residual = T(prepared - result)

Every rank reduces all W payloads (the one-stage exchange, the default).  The result is, bit for bit, what
`codec.dequantize_reduce_tensors` gives for the same payloads, so the torch.distributed path and this one
are interchangeable.

`stages=2` is the reduce-scatter + gather form for many ranks and large tensors (each rank then receives two
payloads' worth of bytes instead of W), four launches of the same two kernels:

  quant_general (scatter)   group g of the payload goes to its owner only (rank g / shard_groups), into slot [me]
                            of the owner's receive region, as a self-contained shard payload; signal
  reduce_general            the owner waits, decodes and sums its W shard payloads, scales: a dense reduced shard
  quant_general (push)      the reduced shard, quantized again, into slot [me] of every rank's gather region; signal
  reduce_general (gather)   wait, decode group g from its owner's slot, write result and residual = T(prepared - result)

Its result is decode(quant(y)) for y = the one-stage result without error feedback applied twice: the reference's
two-stage rule (ccdl_comm/communication/reduce_scatter_transport.py:186-377) with the general codec.  Stochastic
rounding stays with one stage (its random offsets are tied to the element index in the whole tensor).  Receive regions alternate by epoch parity; the argument for reuse without extra
barriers is the one in `parallel/fused.py`.  `fused=False` keeps the earlier composition of separate
launches (quantize, copy-and-signal, wait, W decodes, scale, residual update) for comparison.
"""

from __future__ import annotations

import torch

from ..config import CompressionConfig
from ..ops import oracle
from ..ops.codec import _DTYPE_CODE, _QUANT_CODE, _seed, is_fast_profile
from ..ops.sizing import estimate_quantized_size
from .peer_memory import PHASE_ALL_GATHER, PHASE_REDUCE_SCATTER, PeerGroup


def _round_up(value: int, align: int) -> int:
    return -(-value // align) * align


class GeneralPeerWorkspace:
    """Symmetric regions + one signal channel for general-profile tensors of up to `max_numel` elements."""

    def __init__(self, group: PeerGroup, *, dtype: str, config: CompressionConfig, max_numel: int,
                 max_blocks: int = 0, fused: bool = True) -> None:
        if is_fast_profile(config):
            raise ValueError("linear / top-k 0 / deterministic profiles are served by FusedWorkspace")
        self.group, self.dtype, self.config = group, dtype, config
        self.max_numel, self.max_blocks, self.fused = int(max_numel), int(max_blocks), bool(fused)
        self.ext = group._ext
        self._torch_dtype = oracle.TORCH_DTYPES[dtype]
        self.slot_bytes = self.payload_bytes(dtype, config, self.max_numel)
        self.stage_off = group.alloc(self.slot_bytes)
        self.recv_off = [group.alloc(self.slot_bytes * group.world_size) for _ in range(2)]
        self.channel = group.new_channel()
        self.launches = 0
        self.gather_off: list[int] | None = None          # two-stage only: reserved on first use
        self._shard: torch.Tensor | None = None           # two-stage only: this rank's dense reduced shard

    @staticmethod
    def payload_bytes(dtype: str, config: CompressionConfig, numel: int) -> int:
        return _round_up(estimate_quantized_size(max(1, numel), dtype=dtype, config=config).quantized_bytes, 256)

    @staticmethod
    def required_bytes(world_size: int, dtype: str, config: CompressionConfig, max_numel: int) -> int:
        one_stage = GeneralPeerWorkspace.payload_bytes(dtype, config, max_numel) * (1 + 2 * world_size) + 8 * 512
        shard_slot = GeneralPeerWorkspace.payload_bytes(dtype, config, GeneralPeerWorkspace.shard_numel(
            world_size, config, max_numel))
        return one_stage + 2 * world_size * shard_slot + 4 * 512          # + the two gather regions of stages=2

    @staticmethod
    def shard_numel(world_size: int, config: CompressionConfig, numel: int) -> int:
        """Elements of one rank's shard: whole groups, eight at a time (the scale region of a planar shard payload
        then starts on a 16-byte boundary for every code width)."""

        groups = -(-max(1, numel) // config.group_size)
        return _round_up(-(-groups // world_size), 8) * config.group_size

    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None, *, residual: torch.Tensor | None = None,
                   update_residual: bool = True, op: str = "mean", stages: int = 1) -> torch.Tensor:
        """Compressed all-reduce of `x` into `out` (default: in place); `residual` as in `FusedWorkspace`
        with the reference's rule (residual = T(prepared - result)).  `stages=2`: reduce-scatter + gather."""

        if op not in ("mean", "sum"):
            raise ValueError(f"unsupported reduce op {op!r}")
        if stages not in (1, 2):
            raise ValueError("stages must be 1 or 2")
        if stages == 2 and (self.config.stochastic or not self.fused):
            raise ValueError("the two-stage form needs the fused kernels and deterministic rounding")
        n = x.numel()
        if n > self.max_numel:
            raise ValueError(f"tensor has {n} elements, workspace holds {self.max_numel}")
        if x.dtype != self._torch_dtype or not x.is_contiguous():
            raise TypeError(f"workspace was built for contiguous {self.dtype} tensors")
        target = x if out is None else out
        if n == 0:
            return target
        g, cfg, ext = self.group, self.config, self.ext
        W, me = g.world_size, g.rank
        nbytes = estimate_quantized_size(n, dtype=self.dtype, config=cfg).quantized_bytes
        epoch = g.next_epoch(self.channel)
        region = self.recv_off[epoch & 1]
        flat = x.reshape(-1)
        res = None if residual is None else residual.reshape(-1)
        keep = res if (res is not None and update_residual) else None      # `prepared` is parked here
        out_flat = target.reshape(-1)
        dst = [g.addr(d, region + me * self.slot_bytes) for d in range(W)]
        if stages == 2:
            return self._two_stage(flat, out_flat, res, keep, n, epoch, region, dst, op, target)
        if self.fused:
            ext.quant_general_push(flat, res, keep, dst, cfg.group_size, cfg.bit, cfg.topk, _QUANT_CODE[cfg.quant_type],
                                   cfg.stochastic, cfg.compact, _seed() if cfg.stochastic else 0,
                                   g.signal_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks)
            ext.reduce_general([g.local_ptr + region + r * self.slot_bytes for r in range(W)], out_flat, cfg.group_size,
                               cfg.bit, cfg.topk, _QUANT_CODE[cfg.quant_type], cfg.compact,
                               1.0 / W if (op == "mean" and W > 1) else 1.0, keep, keep,
                               g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks)
            self.launches += 2
            return target
        payload = g.local_view(self.stage_off, nbytes)
        ext.quant_general(flat, res, keep, payload, cfg.group_size, cfg.bit, cfg.topk, _QUANT_CODE[cfg.quant_type],
                          cfg.stochastic, cfg.compact, _seed() if cfg.stochastic else 0)
        ext.push_bytes(g.local_ptr + self.stage_off, _round_up(nbytes, 16), dst, None,
                       g.signal_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks)
        ext.wait_signal(g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), None)
        for r in range(W):
            slot = g.local_view(region + r * self.slot_bytes, nbytes)
            ext.dequant_general(slot, out_flat, cfg.group_size, cfg.bit, cfg.topk, _QUANT_CODE[cfg.quant_type],
                                cfg.compact, r > 0)
        if op == "mean" and W > 1:
            ext.scale_inplace(out_flat, 1.0 / W)
        if keep is not None:
            ext.error_feedback_update(keep, out_flat, keep)
        self.launches += 3 + W + (1 if op == "mean" and W > 1 else 0) + (1 if keep is not None else 0)
        return target

    def _two_stage(self, flat, out_flat, res, keep, n: int, epoch: int, region: int, dst: list[int], op: str, target):
        g, cfg, ext = self.group, self.config, self.ext
        W, me = g.world_size, g.rank
        code = _QUANT_CODE[cfg.quant_type]
        shard_numel = self.shard_numel(W, cfg, n)
        shard_groups = shard_numel // cfg.group_size
        shard_slot = self.payload_bytes(self.dtype, cfg, self.shard_numel(W, cfg, self.max_numel))
        if self.gather_off is None:           # symmetric: every rank reserves them in its first two-stage call
            self.gather_off = [g.alloc(shard_slot * W) for _ in range(2)]
        if self._shard is None or self._shard.numel() < shard_numel or self._shard.device != flat.device:
            self._shard = torch.zeros(self.shard_numel(W, cfg, self.max_numel), dtype=self._torch_dtype, device=flat.device)
        lo = me * shard_numel
        valid = max(0, min(n, lo + shard_numel) - lo)
        shard = self._shard[:shard_numel]
        if valid < shard_numel:
            shard[valid:].zero_()             # what lies past the tensor's end is quantized as zeros
        gather = self.gather_off[epoch & 1]
        # reduce-scatter: my shard r of the payload goes to rank r's slot [me]; then every owner reduces its slots
        ext.quant_general_push(flat, res, keep, dst, cfg.group_size, cfg.bit, cfg.topk, code, False, cfg.compact, 0,
                               g.signal_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks, shard_groups)
        if valid:
            ext.reduce_general([g.local_ptr + region + r * self.slot_bytes for r in range(W)], shard[:valid],
                               cfg.group_size, cfg.bit, cfg.topk, code, cfg.compact,
                               1.0 / W if (op == "mean" and W > 1) else 1.0, None, None,
                               g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks, shard_groups, 0)
        else:       # a shard wholly past the tensor's end: nothing to reduce, but the scatter's signals are consumed
            ext.wait_signal(g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), None)
        # gather: the reduced shard, quantized again, into slot [me] of every rank; then everybody decodes
        ext.quant_general_push(shard, None, None, [g.addr(d, gather + me * shard_slot) for d in range(W)],
                               cfg.group_size, cfg.bit, cfg.topk, code, False, cfg.compact, 0,
                               g.signal_all(self.channel, PHASE_ALL_GATHER, epoch), self.max_blocks, 0)
        ext.reduce_general([g.local_ptr + gather + r * shard_slot for r in range(W)], out_flat, cfg.group_size, cfg.bit,
                           cfg.topk, code, cfg.compact, 1.0, keep, keep,
                           g.wait_all(self.channel, PHASE_ALL_GATHER, epoch), self.max_blocks, 0, shard_groups)
        self.launches += 4
        return target
