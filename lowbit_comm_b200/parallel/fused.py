"""Host drivers of the fused compression + NVLink collectives.

One `FusedWorkspace` owns symmetric receive regions inside a `PeerGroup` arena
and one signal channel.  Its methods only enqueue kernels on the current CUDA
stream; nothing here synchronises with the host.

Two-stage all-reduce (W >= 3 above a few MiB), per rank:
  K1 quant_push/scatter : x (+residual) -> int8 groups; group g goes to the rank
                          owning shard g // shard_groups, into that rank's RS
                          region slot [me]; then signals RS[me] on every rank
  K2 reduce             : waits RS[0..W); dequantizes the W slots of its shard,
                          sums in fp32, scales, requantizes the shard into its OWN
                          AG region (a self-contained payload); then signals AG[me]
  K3 reduce (gather)    : waits AG[0..W); loads shard s from rank s's AG region
                          (peer loads over NVLink), decodes into `out`; updates the
                          residual
(`set_gather_mode("push")`: K2 stores its shard into every rank's AG region instead
and K3 reads only local memory.)
One-stage all-reduce (W <= 2, small tensors): K1 broadcasts the whole payload to
every rank's gather region slot [me]; one reduce kernel sums the W slots.

Why reuse of the regions is safe without extra barriers: all ranks enqueue the
same kernel sequence on one in-order stream.  K3(t) of a rank finishes only
after every peer's K2(t) signalled, so by the time the rank's K1(t+1) overwrites
a peer's RS slot that peer has finished reading it.  A rank overwrites its own AG
region in K2(t+1), which waits for every peer's K1(t+1) signal, and a peer enqueues
K1(t+1) after its K3(t), the kernel that read this rank's AG region (push mode: the
same argument with "writes the peers' AG regions").  Regions that are read by a
kernel not followed by such a barrier (gather region, RS region used by
reduce-scatter alone) are double buffered by epoch parity, which the same argument
makes sufficient.

Engines.  The default engine ("pipe") runs the whole all-reduce as ONE persistent kernel
(`ops/csrc/pipe_kernels.cu`): every rank quantizes into its own arena, shard owners pull rows from all
ranks with bulk asynchronous loads, reduce and requantize them, and every rank pulls and decodes the
reduced rows; per-chunk epoch flags let the three phases of neighbouring chunks overlap inside the
launch.  Its regions: the own quantized payload (written by this rank, read by the peers' REDUCE
rows), the own reduced shard (read by the peers' DECODE rows) and a control block of flags and
counters.  Reuse without extra barriers: a rank's kernel only ends after it has decoded every chunk,
i.e. after every owner finished reducing (= reading this rank's payload); and a rank requantizes
chunk c of collective t+1 only after every peer's QUANT flag of t+1, which a peer raises after its
kernel of collective t (the one that read this rank's reduced shard) has ended.
The "legacy" engine is the K1/K2/K3 sequence described above; reduce-scatter and all-gather use it.

This replaces the reference's quantize -> NCCL all_to_all / all_gather ->
dequantize chains (ccdl_comm/communication/reduce_scatter_transport.py:186-377,
ccdl_comm/collectives/all_reduce.py:158-271).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ..config import CompressionConfig
from ..core.chunking import GroupShardPlan
from ..ops import oracle
from ..ops.codec import _DTYPE_CODE, is_fast_profile
from ..ops.sizing import dtype_bytes
from .peer_memory import PHASE_ALL_GATHER, PHASE_REDUCE_SCATTER, PeerGroup

ALIGN_GROUPS = 8
MAX_CHUNKS = 8          # pipeline depth of the native launcher (one flag channel per chunk)


def _round_up(value: int, align: int) -> int:
    return -(-value // align) * align


def _chunk_slack(world_size: int, config: CompressionConfig) -> int:
    """Extra elements of capacity: every chunk of a pipelined call rounds its regions up separately."""

    return 2 * MAX_CHUNKS * world_size * ALIGN_GROUPS * config.group_size + MAX_CHUNKS * 256 * 8


def _current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


@dataclass(frozen=True)
class FusedGeometry:
    numel: int
    world_size: int
    group_size: int
    value_bytes: int     # per group
    scale_bytes: int     # per group
    shard_groups: int
    num_groups: int

    @property
    def group_bytes(self) -> int:
        return self.value_bytes + self.scale_bytes

    @property
    def total_groups(self) -> int:
        return self.shard_groups * self.world_size

    @property
    def full_groups(self) -> int:
        """Groups of a whole-tensor payload, padded to the alignment unit."""

        return _round_up(self.num_groups, ALIGN_GROUPS)

    @property
    def shard_numel(self) -> int:
        return self.shard_groups * self.group_size

    def shard_valid_numel(self, rank: int) -> int:
        lo = rank * self.shard_numel
        return max(0, min(self.numel, lo + self.shard_numel) - lo)


def geometry(numel: int, world_size: int, dtype: str, config: CompressionConfig) -> FusedGeometry:
    plan = GroupShardPlan.build(numel, world_size, config.group_size, ALIGN_GROUPS)
    return FusedGeometry(numel, world_size, config.group_size, config.group_size * config.bit // 8,
                         dtype_bytes(dtype), plan.shard_groups, plan.num_groups)


def default_stages(world_size: int, nbytes: int, multicast: bool = False) -> int:
    """One-stage (every rank reduces W payloads) or two-stage (scatter, reduce, gather) all-reduce.

    Measured on B200 (bf16, int8 group 64): one stage wins while launches and signal round trips
    dominate; the crossover sits near 16-32 MiB on 4 GPUs and 8 MiB on 8 GPUs, i.e. where the
    tensor is about 64 MiB / W (twice that when the broadcast leaves through the NVLink multicast
    mapping).  Above it the (W - 1) payloads per rank lose to the 2 (W - 1) / W of the two-stage
    path.  Two ranks move the same bytes either way.
    """

    if world_size <= 2:
        return 1
    budget = (128 << 20) if multicast else (64 << 20)
    return 1 if nbytes * world_size <= budget else 2


class FusedWorkspace:
    """Symmetric regions + channel for tensors of up to `max_numel` elements."""

    def __init__(self, group: PeerGroup, *, dtype: str, config: CompressionConfig, max_numel: int,
                 max_blocks: int = 0, with_gather_region: bool | None = None, engine: str | None = None) -> None:
        if not is_fast_profile(config):
            raise ValueError("fused collectives serve linear / top-k 0 / deterministic profiles")
        self.group = group
        self.dtype = dtype
        self.config = config
        self.max_numel = int(max_numel)
        self.max_blocks = int(max_blocks)
        self.ext = group._ext
        self._torch_dtype = oracle.TORCH_DTYPES[dtype]
        cap = geometry(self.max_numel + _chunk_slack(group.world_size, config), group.world_size, dtype, config)
        self.cap = cap
        W = group.world_size
        self.shard_stride = _round_up(max(cap.shard_groups, ALIGN_GROUPS) * cap.group_bytes, 256)
        self.rs_bytes = W * self.shard_stride
        self.ag_bytes = _round_up(max(cap.total_groups, ALIGN_GROUPS) * cap.group_bytes, 256)
        self.gather_stride = _round_up(max(cap.full_groups, ALIGN_GROUPS) * cap.group_bytes, 256)
        self.rs_off: list[int] | None = None       # legacy regions are reserved on first use (`_ensure_legacy`)
        self.ag_off: int | None = None
        self.gather_off: list[int] | None = None
        self._want_gather = bool(with_gather_region or (with_gather_region is None and W <= 2))
        # pipelined engine: own quantized payload, own reduced shard, control block
        self.engine = (engine or os.environ.get("LBC_ENGINE", "auto")).lower()
        if self.engine not in ("auto", "pipe", "legacy"):
            raise ValueError("engine must be 'auto', 'pipe' or 'legacy'")
        if not hasattr(self.ext, "PipeAllReducePlan"):
            self.engine = "legacy"
        # "auto": the single persistent kernel up to this many bytes, the kernel sequence above (measured on
        # 4 x B200: the single kernel is ahead up to 128 MiB, by a fifth around 32 MiB, and 4-9 % behind from 256 MiB)
        self.pipe_max_bytes = int(float(os.environ.get("LBC_PIPE_MAX_MIB", "192")) * (1 << 20))
        self.gate = False                           # rendezvous kernel in front of the single persistent kernel
        self._pipe = None
        if self.engine in ("auto", "pipe"):
            self._build_pipe()
        else:
            self._ensure_legacy()
        self.channels = [group.new_channel() for _ in range(MAX_CHUNKS)]
        self.channel = self.channels[0]
        self.launches = 0
        self.phase_timer = None   # set to a utils.tracing.PhaseTimer to time K1/K2/K3 separately
        # Real process groups launch through the native plan (one binding crossing per collective);
        # emulated single-GPU groups keep the Python path so that launches can be interleaved by phase.
        self._native = None
        # Chunk pipelining is off by default: measured on 2 x B200 it was slower than the plain sequence
        # (persistent grids of neighbouring chunks do not interleave; one-tile blocks pay a system-scope
        # fence each).  `set_chunking` turns it on for experiments.
        self.min_chunk_bytes, self.max_chunks = 16 << 20, 1
        # multimem stores serve the one-stage broadcast; the two-stage broadcast keeps unicast stores (faster
        # above 64 MiB on 8 GPUs) unless this is set before the first collective
        self.multicast_in_reduce_stage = os.environ.get("LBC_MULTICAST_REDUCE", "0") == "1"
        # Gather stage of the two-stage path: True = every rank's decode kernel loads the reduced shards
        # from their owners' memory (the NVLink crossing hides behind decode + error feedback; measured
        # 600 GB/s per GPU with the local work fully overlapped); False = the reduce stage stores its shard
        # into every rank's gather region.
        self.pull_gather = os.environ.get("LBC_GATHER", "pull") != "push"
        # Decode stage with several tiles of peer loads in flight per thread (2 or 4); process-wide, off unless
        # asked for.  `ext.set_gather_prefetch` changes it at run time.
        prefetch = os.environ.get("LBC_GATHER_PREFETCH")
        if prefetch is not None and hasattr(self.ext, "set_gather_prefetch"):
            self.ext.set_gather_prefetch(int(prefetch))
        if self.rs_off is not None:
            self._build_native()

    # -- pipelined engine -------------------------------------------------------
    @staticmethod
    def pipe_region_bytes(world_size: int, dtype: str, config: CompressionConfig, max_numel: int) -> tuple[int, int]:
        """(own payload bytes, reduced shard bytes) the pipelined engine needs for `max_numel` elements."""

        group_bytes = config.group_size * config.bit // 8 + dtype_bytes(dtype)
        groups = -(-max(1, max_numel) // config.group_size)
        one = _round_up(_round_up(groups, ALIGN_GROUPS) * group_bytes, 256)
        shard_groups = _round_up(-(-groups // world_size), ALIGN_GROUPS)
        two = world_size * _round_up(shard_groups * group_bytes, 256)
        return max(one, two), _round_up(shard_groups * group_bytes, 256)

    def _pipe_numel(self) -> int:
        """Elements the single-kernel engine has to hold: everything, or in "auto" what fits its size limit."""

        if self.engine != "auto":
            return self.max_numel
        return min(self.max_numel, self.pipe_max_bytes // dtype_bytes(self.dtype))

    def _build_pipe(self) -> None:
        group = self.group
        self.pipe_numel = self._pipe_numel()
        q_bytes, ag_bytes = self.pipe_region_bytes(group.world_size, self.dtype, self.config, self.pipe_numel)
        self.pipe_q_off, self.pipe_q_bytes = group.alloc(q_bytes), q_bytes
        self.pipe_ag_off, self.pipe_ag_bytes = group.alloc(ag_bytes), ag_bytes
        self.pipe_ctl_off = group.alloc(int(self.ext.PIPE_CTL_BYTES))
        self._pipe = self.ext.PipeAllReducePlan(
            _DTYPE_CODE[self.dtype], self.config.group_size, self.config.bit, group.rank, list(group.peer_ptrs),
            self.pipe_q_off, q_bytes, self.pipe_ag_off, ag_bytes, self.pipe_ctl_off, group.timeout_ns,
            group.status_device, self.max_blocks, self.pipe_numel)
        depth = os.environ.get("LBC_PIPE_RING")
        if depth:
            self._pipe.set_ring_depth(int(depth))

    def set_engine(self, engine: str) -> None:
        """"pipe": one persistent kernel per all-reduce; "legacy": the K1/K2/K3 kernel sequence; "auto": the
        single kernel up to `pipe_max_bytes`, the sequence above."""

        if engine not in ("auto", "pipe", "legacy"):
            raise ValueError("engine must be 'auto', 'pipe' or 'legacy'")
        if engine != "legacy" and not hasattr(self.ext, "PipeAllReducePlan"):
            raise ValueError("this build has no single-kernel engine")
        previous, self.engine = self.engine, engine
        if engine != "legacy" and (self._pipe is None or self.pipe_numel < self._pipe_numel()):
            self._build_pipe()                      # first use, or "pipe" after "auto": regions for every size
        if engine == "legacy":
            self._ensure_legacy()
        del previous

    def reset_pipe_control(self) -> None:
        """After a failed collective: zero this rank's local counters of the pipelined engine."""

        if self._pipe is not None:
            local = int(self.ext.PIPE_CTL_LOCAL)
            with torch.cuda.device(self.group.device):
                self.ext.memset_async(self.group.local_ptr + self.pipe_ctl_off + local, 0,
                                      int(self.ext.PIPE_CTL_BYTES) - local)

    def _ensure_legacy(self) -> None:
        if self.rs_off is not None:
            return
        group = self.group
        self.rs_off = [group.alloc(self.rs_bytes), group.alloc(self.rs_bytes)]
        self.ag_off = group.alloc(self.ag_bytes)
        if self._want_gather:
            self._ensure_gather()
        if hasattr(self, "channels"):
            self._build_native()

    def _build_native(self) -> None:
        group = self.group
        if group.process_group is None or not hasattr(self.ext, "FusedAllReducePlan"):
            return
        from .peer_memory import COUNTER_OFFSET

        self._native = self.ext.FusedAllReducePlan(
            _DTYPE_CODE[self.dtype], self.config.group_size, self.config.bit, group.rank, list(group.peer_ptrs),
            list(self.rs_off), self.rs_bytes, self.ag_off, self.ag_bytes, list(self.gather_off or []),
            group.world_size * self.gather_stride, list(self.channels), COUNTER_OFFSET, group.timeout_ns,
            group.status_device, self.max_blocks, self.max_numel)
        self._native.set_chunking(self.min_chunk_bytes, self.max_chunks)
        self._native.set_multicast(group.multicast_ptr, self.multicast_in_reduce_stage)
        self._native.set_pull_gather(self.pull_gather)

    def set_gather_mode(self, mode: str) -> None:
        """"pull" (default) or "push": how the reduced shards reach the other ranks (see `pull_gather`)."""

        if mode not in ("pull", "push"):
            raise ValueError("gather mode must be 'pull' or 'push'")
        self.pull_gather = mode == "pull"
        if self._native is not None:
            self._native.set_pull_gather(self.pull_gather)

    def set_chunking(self, min_chunk_bytes: int, max_chunks: int = MAX_CHUNKS) -> None:
        """Tensors of at least 2 x `min_chunk_bytes` are pipelined in up to `max_chunks` chunks."""

        self.min_chunk_bytes, self.max_chunks = int(min_chunk_bytes), int(max_chunks)
        if self._native is not None:
            self._native.set_chunking(self.min_chunk_bytes, self.max_chunks)

    @staticmethod
    def required_bytes(world_size: int, dtype: str, config: CompressionConfig, max_numel: int,
                       with_gather_region: bool, engine: str = "both") -> int:
        """Arena bytes one workspace may reserve: "pipe" (all-reduce only), "legacy", or "both"."""

        total = 0
        if engine in ("pipe", "both"):
            q_bytes, ag_bytes = FusedWorkspace.pipe_region_bytes(world_size, dtype, config, max_numel)
            total += q_bytes + ag_bytes + 4096 + 4 * 512
        if engine in ("legacy", "both"):
            cap = geometry(max_numel + _chunk_slack(world_size, config), world_size, dtype, config)
            shard = _round_up(max(cap.shard_groups, ALIGN_GROUPS) * cap.group_bytes, 256)
            total += 2 * world_size * shard + _round_up(max(cap.total_groups, ALIGN_GROUPS) * cap.group_bytes, 256)
            if with_gather_region:
                total += 2 * world_size * _round_up(max(cap.full_groups, ALIGN_GROUPS) * cap.group_bytes, 256)
            total += 32 * 256   # rounding and canaries of the five regions
        return total

    def _ensure_gather(self) -> list[int]:
        if self.gather_off is None:
            size = self.group.world_size * self.gather_stride
            self.gather_off = [self.group.alloc(size), self.group.alloc(size)]
            if getattr(self, "_native", None) is not None:
                self._build_native()
        return self.gather_off

    def _pipe_all_reduce(self, x, out, residual, update_residual: bool, scale: float, stages: int, ef_mode: str):
        n = x.numel()
        if n > self.max_numel or x.dtype != self._torch_dtype or not x.is_contiguous():
            self._geom(x)  # raises the precise error
        target = x if out is None else out
        if n == 0:
            return target
        if target.dtype != x.dtype or target.numel() != n or not target.is_contiguous():
            raise ValueError("out must be a contiguous tensor of the input's dtype and size")
        if residual is not None and (residual.dtype != x.dtype or residual.numel() != n or not residual.is_contiguous()):
            raise ValueError("residual must be a contiguous tensor of the input's dtype and size")
        epoch = self.group.next_epoch(self.channel)
        args = (self._pipe, x.data_ptr(), target.data_ptr(), 0 if residual is None else residual.data_ptr(), n, stages,
                scale, bool(update_residual), ef_mode == "local", epoch, _current_stream_ptr(x.device))
        if self.group.process_group is None and self.group.world_size > 1:
            # emulated ranks on one GPU: one launch per phase, so that the ranks can be interleaved by phase
            phases = [self.ext.PIPE_QUANT, self.ext.PIPE_REDUCE] + ([self.ext.PIPE_DECODE] if stages == 2 else [])
            for mask in phases:
                self.ext.pipe_all_reduce(*args, int(mask), False)
                self.launches += 1
        else:
            done = self.ext.pipe_all_reduce(*args, int(self.ext.PIPE_ALL), bool(self.gate))
            self.launches += 1 if done is None else done      # None: a recorder deferred the launch
        return target

    # -- helpers ---------------------------------------------------------------
    def _geom(self, x: torch.Tensor) -> FusedGeometry:
        if x.numel() > self.max_numel:
            raise ValueError(f"tensor has {x.numel()} elements, workspace holds {self.max_numel}")
        if oracle.dtype_name(x) != self.dtype:
            raise TypeError(f"workspace was built for {self.dtype}")
        if not x.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return geometry(x.numel(), self.group.world_size, self.dtype, self.config)

    @property
    def _code(self) -> int:
        return _DTYPE_CODE[self.dtype]

    def _scale(self, op: str) -> float:
        if op == "mean":
            return 1.0 / self.group.world_size
        if op == "sum":
            return 1.0
        raise ValueError(f"unsupported reduce op {op!r}")

    # -- kernels ---------------------------------------------------------------
    def _k1_scatter(self, x, residual, prepared_out, local_ef_out, geo: FusedGeometry, epoch: int, parity: int):
        g, me = self.group, self.group.rank
        dst = [g.addr(d, self.rs_off[parity] + me * self.shard_stride) for d in range(g.world_size)]
        self.ext.quant_push(x, residual, prepared_out, local_ef_out, dst, self.ext.PUSH_SCATTER,
                            geo.shard_groups, geo.shard_groups, 0, geo.group_size, self.config.bit,
                            g.signal_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks)
        self.launches += 1

    def _k2_reduce(self, geo: FusedGeometry, epoch: int, parity: int, scale: float, out, broadcast: bool):
        g, me = self.group, self.group.rank
        src = [g.local_ptr + self.rs_off[parity] + r * self.shard_stride for r in range(g.world_size)]
        signal = g.signal_all(self.channel, PHASE_ALL_GATHER, epoch) if broadcast else None
        dst, dst_layout, dst_offset, mc = [], geo.total_groups, me * geo.shard_groups, 0
        if broadcast and self.pull_gather:
            # the reduced shard stays here as a self-contained payload; peers load it in their K3
            dst, dst_layout, dst_offset = [g.local_ptr + self.ag_off], geo.shard_groups, 0
        elif broadcast:
            dst = [g.addr(d, self.ag_off) for d in range(g.world_size)]
            mc = g.multicast_addr(self.ag_off) if self.multicast_in_reduce_stage else 0
        self.ext.wait_signal(g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), None)
        self.launches += 1
        self.ext.reduce(src, geo.shard_groups, 0, False, geo.shard_valid_numel(me), self._code, geo.group_size,
                        self.config.bit, scale, out, False, None, None, dst, dst_layout, dst_offset, signal,
                        g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks, mc)
        self.launches += 1

    def _k3_gather(self, geo: FusedGeometry, epoch: int, out, prepared, residual_out):
        g = self.group
        self.ext.wait_signal(g.wait_all(self.channel, PHASE_ALL_GATHER, epoch), None)
        self.launches += 1
        if self.pull_gather:
            src, layout, shard_groups = [g.addr(r, self.ag_off) for r in range(g.world_size)], geo.shard_groups, \
                geo.shard_groups
        else:
            src, layout, shard_groups = [g.local_ptr + self.ag_off], geo.total_groups, 0
        self.ext.reduce(src, layout, 0, False, geo.numel, self._code, geo.group_size, self.config.bit, 1.0, out,
                        False, prepared, residual_out, [], 0, 0, None,
                        g.wait_all(self.channel, PHASE_ALL_GATHER, epoch), self.max_blocks, 0, shard_groups,
                        g.rank if shard_groups else 0)
        self.launches += 1

    def _k1_broadcast(self, x, residual, prepared_out, local_ef_out, geo: FusedGeometry, epoch: int, parity: int):
        g, me = self.group, self.group.rank
        region = self._ensure_gather()[parity]
        dst = [g.addr(d, region + me * self.gather_stride) for d in range(g.world_size)]
        self.ext.quant_push(x, residual, prepared_out, local_ef_out, dst, self.ext.PUSH_BROADCAST, 0,
                            geo.full_groups, 0, geo.group_size, self.config.bit,
                            g.signal_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks,
                            g.multicast_addr(region + me * self.gather_stride))
        self.launches += 1

    # -- collectives -------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None, *, residual: torch.Tensor | None = None,
                   update_residual: bool = True, op: str = "mean", stages: int | None = None,
                   ef_mode: str = "reference") -> torch.Tensor:
        """Compressed all-reduce of `x` into `out` (default: in place).

        `residual` is added before quantization.  With `update_residual` it is
        rewritten: ef_mode="reference" stores T(prepared - result) (the rule of
        ccdl_comm/communication/ddp_hook.py:268-277), ef_mode="local" stores this
        rank's own quantization error.
        """

        through_pipe, stages = self.route(x.numel(), x.element_size(), stages)
        scale = self._scale(op)
        if ef_mode not in ("reference", "local"):
            raise ValueError("ef_mode must be 'reference' or 'local'")
        if through_pipe and self.phase_timer is None:
            return self._pipe_all_reduce(x, out, residual, update_residual, scale, stages, ef_mode)
        self._ensure_legacy()
        if self._native is not None and self.phase_timer is None:
            # hot path: one binding crossing; geometry is recomputed natively
            n = x.numel()
            if n > self.max_numel or x.dtype != self._torch_dtype or not x.is_contiguous():
                self._geom(x)  # raises the precise error
            if n == 0:
                return x if out is None else out
            if stages == 1:
                self._ensure_gather()
            epoch = self.group.next_epoch(self.channel)
            target = x if out is None else out
            self.launches += self._native.all_reduce(
                x.data_ptr(), target.data_ptr(), 0 if residual is None else residual.data_ptr(), n, stages, scale,
                bool(update_residual), ef_mode == "local", epoch, _current_stream_ptr(x.device))
            return target
        geo = self._geom(x)
        flat = x.reshape(-1)
        out_flat = flat if out is None else out.reshape(-1)
        res = None if residual is None else residual.reshape(-1)
        epoch = self.group.next_epoch(self.channel)
        parity = epoch & 1
        want_ref = res is not None and update_residual and ef_mode == "reference"
        want_local = res is not None and update_residual and ef_mode == "local"
        prepared_out = res if want_ref else None
        local_out = res if want_local else None
        if geo.numel == 0:
            return x if out is None else out
        if stages == 1:
            self._ensure_gather()
        timer = self.phase_timer
        if timer is not None:
            timer.mark("start")
        if stages == 1:
            self._k1_broadcast(flat, res, prepared_out, local_out, geo, epoch, parity)
            if timer is not None:
                timer.mark("k1_quant_push")
            region = self.gather_off[parity]
            src = [self.group.local_ptr + region + r * self.gather_stride for r in range(self.group.world_size)]
            self.ext.wait_signal(self.group.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), None)
            self.launches += 1
            self.ext.reduce(src, geo.full_groups, 0, False, geo.numel, self._code, geo.group_size, self.config.bit,
                            scale, out_flat, False, res if want_ref else None, res if want_ref else None, [], 0, 0,
                            None, self.group.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), self.max_blocks)
            self.launches += 1
            if timer is not None:
                timer.mark("k2_reduce_all")
        else:
            self._k1_scatter(flat, res, prepared_out, local_out, geo, epoch, parity)
            if timer is not None:
                timer.mark("k1_quant_push")
            self._k2_reduce(geo, epoch, parity, scale, None, True)
            if timer is not None:
                timer.mark("k2_reduce_requant_push")
            self._k3_gather(geo, epoch, out_flat, res if want_ref else None, res if want_ref else None)
            if timer is not None:
                timer.mark("k3_gather_decode")
        if timer is not None:
            timer.flush()
        return x if out is None else out

    def route(self, numel: int, element_size: int, stages: int | None = None) -> tuple[bool, int]:
        """(through the single kernel?, stage count) an all-reduce of `numel` elements takes on this workspace.

        "auto" takes the single persistent kernel, except where the kernel sequence measured faster: on two ranks
        (46 vs 50 us at 1 MiB, 155 vs 185 us at 64 MiB) and above the size limit.  Without a requested stage
        count the kernel sequence uses `default_stages`; the single kernel pays less per stage, which moves the
        crossover down: one stage up to 16 MiB / W (4 GPUs: 4 MiB 63 vs 74 us, 8 MiB 103 vs 82 us; 8 GPUs: 2 MiB
        71 vs 79 us, 4 MiB 84 vs 79 us, one stage against two)."""

        world, nbytes = self.group.world_size, numel * element_size
        through_pipe = self.engine == "pipe" or (self.engine == "auto" and world != 2 and numel <= self.pipe_numel)
        if stages is None:
            if through_pipe and world > 2:
                stages = 1 if nbytes * world <= (16 << 20) else 2
            else:
                stages = default_stages(world, nbytes, bool(self.group.multicast_ptr))
        return through_pipe, stages

    def reduce_scatter(self, x: torch.Tensor, out_shard: torch.Tensor, *, residual: torch.Tensor | None = None,
                       update_residual: bool = True, op: str = "mean") -> FusedGeometry:
        """Rank r receives the reduced elements [r*shard_numel, (r+1)*shard_numel).

        `out_shard` holds `shard_numel` elements (group aligned); elements past
        the end of the tensor are zero.  Error feedback, when a residual is
        given, uses this rank's own quantization error.
        """

        self._ensure_legacy()
        geo = self._geom(x)
        if out_shard.numel() != geo.shard_numel:
            raise ValueError(f"out_shard must hold {geo.shard_numel} elements")
        res = None if residual is None else residual.reshape(-1)
        epoch = self.group.next_epoch(self.channel)
        parity = epoch & 1
        valid = geo.shard_valid_numel(self.group.rank)
        flat_out = out_shard.reshape(-1)
        if valid < geo.shard_numel:
            flat_out[valid:].zero_()
        if self._native is not None and self.phase_timer is None and hasattr(self._native, "reduce_scatter"):
            # hot path: one binding crossing for the three launches
            if geo.numel:
                self.launches += self._native.reduce_scatter(
                    x.data_ptr(), flat_out.data_ptr(), 0 if res is None else res.data_ptr(), geo.numel, self._scale(op),
                    bool(update_residual), epoch, _current_stream_ptr(x.device))
            return geo
        self._k1_scatter(x.reshape(-1), res, None, res if (res is not None and update_residual) else None, geo,
                         epoch, parity)
        self._k2_reduce(geo, epoch, parity, self._scale(op), flat_out[:valid] if valid else None, False)
        return geo

    def all_gather(self, x: torch.Tensor, outs: list[torch.Tensor]) -> list[torch.Tensor]:
        """Every rank contributes `x` (same shape everywhere); outs[r] = decode(rank r's payload)."""

        self._ensure_legacy()
        geo = self._geom(x)
        g = self.group
        if len(outs) != g.world_size:
            raise ValueError("one output per rank is required")
        epoch = g.next_epoch(self.channel)
        parity = epoch & 1
        if geo.numel == 0:
            return outs
        self._k1_broadcast(x.reshape(-1), None, None, None, geo, epoch, parity)
        region = self.gather_off[parity]
        self.ext.wait_signal(g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch), None)
        self.launches += 1
        wait = g.wait_all(self.channel, PHASE_REDUCE_SCATTER, epoch)
        step = geo.numel * x.element_size()
        one_buffer = all(o.is_contiguous() and o.dtype == x.dtype and o.numel() == geo.numel and
                         o.data_ptr() == outs[0].data_ptr() + r * step for r, o in enumerate(outs))
        if one_buffer and geo.num_groups == geo.full_groups and geo.numel % geo.group_size == 0:
            # the outputs are rows of one buffer and every payload is a whole number of 8-group units: ONE decode
            # launch reads payload r for the groups of row r (the gather mode of the reduce kernel)
            whole = self.ext.tensor_from_address(outs[0].data_ptr(), step * g.world_size, x.device.index) \
                .view(self._torch_dtype)
            src = [g.local_ptr + region + r * self.gather_stride for r in range(g.world_size)]
            self.ext.reduce(src, geo.full_groups, 0, False, geo.numel * g.world_size, self._code, geo.group_size,
                            self.config.bit, 1.0, whole, False, None, None, [], 0, 0, None, wait, self.max_blocks, 0,
                            geo.full_groups, 0)
            self.launches += 1
            return outs
        for r, out in enumerate(outs):
            self.ext.reduce([g.local_ptr + region + r * self.gather_stride], geo.full_groups, 0, False, geo.numel,
                            self._code, geo.group_size, self.config.bit, 1.0, out.reshape(-1), False, None, None,
                            [], 0, 0, None, wait if r == 0 else None, self.max_blocks)
            self.launches += 1
        return outs


    def gather_shards(self, shard: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Compressed all-gather of reduced shards, straight into one tensor (the closing stage of the
        hierarchical all-reduce): rank r contributes `shard`, the `shard_numel` elements it owns of a tensor of
        `out.numel()` elements (the geometry of `reduce_scatter`); every rank ends up with
        out = concat(decode(encode(shard_0)), decode(encode(shard_1)), ...)[:numel].

        Two launches and a one-warp gate: the shard is quantized into this rank's own region, and one decode
        kernel loads every owner's payload from that owner's memory and writes the output in place -- no list
        of W tensors, no concatenation, no copy.
        """

        self._ensure_legacy()
        g = self.group
        geo = self._geom(out)
        flat_out = out.reshape(-1)
        if shard.numel() != geo.shard_numel or shard.dtype != out.dtype or not shard.is_contiguous():
            raise ValueError(f"shard must be a contiguous tensor of {geo.shard_numel} elements of the output's dtype")
        if geo.numel == 0:
            return out
        epoch = g.next_epoch(self.channel)
        # Own payload of shard_groups groups in this rank's all-gather region; the W flags of the all-gather
        # phase tell every rank that every payload is complete.  Two halves of the region alternate by epoch
        # parity: a peer may still be decoding the previous payload when this rank writes the next one, and
        # by the time the half is reused that peer has signalled once more, i.e. finished that decode.
        half = _round_up(geo.shard_groups * geo.group_bytes, 256) if g.world_size > 1 else 0
        if 2 * half > self.ag_bytes:
            raise ValueError("workspace too small to gather shards of this tensor")
        region = self.ag_off + (epoch & 1) * half
        self.ext.quant_push(shard.reshape(-1), None, None, None, [g.local_ptr + region], self.ext.PUSH_BROADCAST,
                            0, geo.shard_groups, 0, geo.group_size, self.config.bit,
                            g.signal_all(self.channel, PHASE_ALL_GATHER, epoch), self.max_blocks, 0)
        self.ext.wait_signal(g.wait_all(self.channel, PHASE_ALL_GATHER, epoch), None)
        src = [g.addr(r, region) for r in range(g.world_size)]
        self.ext.reduce(src, geo.shard_groups, 0, False, geo.numel, self._code, geo.group_size, self.config.bit, 1.0,
                        flat_out, False, None, None, [], 0, 0, None, g.wait_all(self.channel, PHASE_ALL_GATHER, epoch),
                        self.max_blocks, 0, geo.shard_groups, g.rank)
        self.launches += 3
        return out


def run_loopback(workspaces: list[FusedWorkspace], method: str, per_rank_args: list[tuple],
                 per_rank_kwargs: list[dict] | None = None, **kwargs) -> list:
    """Single-GPU emulation: run one collective for all emulated ranks, phase by phase.

    Kernels that wait must start only after the kernels that signal them were
    enqueued for *all* emulated ranks (one stream, one GPU), so the launches of
    the ranks are interleaved by phase rather than run rank after rank.
    """

    extra = per_rank_kwargs or [{}] * len(workspaces)
    plans = [_PhasedCall(ws, method, args, {**kwargs, **kw}) for ws, args, kw in zip(workspaces, per_rank_args, extra)]
    depth = max(len(p.steps) for p in plans)
    for level in range(depth):
        for p in plans:
            if level < len(p.steps):
                p.steps[level]()
    return [p.result for p in plans]


class _PhasedCall:
    """Records the kernel launches of one collective call so they can be replayed by phase."""

    def __init__(self, ws: FusedWorkspace, method: str, args: tuple, kwargs: dict) -> None:
        self.steps: list = []
        recorder = _Recorder(ws.ext, self.steps)
        real = ws.ext
        ws.ext = recorder
        try:
            self.result = getattr(ws, method)(*args, **kwargs)
        finally:
            ws.ext = real


class _Recorder:
    def __init__(self, ext, steps: list) -> None:
        self._ext = ext
        self._steps = steps

    def __getattr__(self, name):
        attr = getattr(self._ext, name)
        if name in ("quant_push", "reduce", "push_bytes", "wait_signal", "pipe_all_reduce", "quant_general",
                    "dequant_general", "scale_inplace", "error_feedback_update", "quant_general_push",
                    "reduce_general"):
            def defer(*a, **k):
                self._steps.append(lambda: attr(*a, **k))
            return defer
        return attr
