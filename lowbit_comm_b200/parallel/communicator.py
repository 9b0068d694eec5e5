"""Per-process-group communicator: owns the peer arena, the fused workspaces,
the side stream and the torch.distributed fallbacks, and runs every compressed
collective of the public API.

Role parity: this one object replaces the reference's per-call plumbing —
`compile_cuda_shortcut` building a fresh registry on every call
(ccdl_comm/cuda/shortcut.py:18-59), the transport factories
(communication/reduce_scatter_transport.py, topology_transport.py,
hierarchical_transport.py) and the executors (cuda/executors.py:30-220).
Strategy names of the reference map onto two data paths:

    all_gather                      -> one-stage (quantize once, every rank reduces W payloads)
    reduce_scatter/topology/ring/   -> two-stage (scatter, reduce + requantize, gather)
    tree/p2p/overlap-*
    hierarchical                    -> intra-group reduce-scatter, inter-group all-reduce, intra-group gather
    native_nccl                     -> plain torch.distributed all_reduce

On CUDA tensors with peer access the fused kernels move the data; otherwise the
same algorithms run over torch.distributed with the codec facade (CPU/gloo too).
"""

from __future__ import annotations

import contextlib
import os
import threading
from importlib import import_module
from typing import Any

from ..config import CompressionConfig
from ..core.chunking import GroupShardPlan
from ..core.info import ExecutionInfo
from ..core.shard import ReducedShard
from ..core.work import ImmediateWork
from ..exceptions import CCDLUnavailableError, UnsupportedCollective
from ..ops import codec
from ..ops.loader import load_cuda_extension
from ..ops.sizing import estimate_quantized_size
from ..utils import tracing
from .payload import payload_buffer
from .torch_transport import make_torch_all_gather, make_torch_all_to_all, make_torch_tensor_all_reduce

TWO_STAGE = frozenset({"reduce_scatter", "topology", "ring", "tree", "p2p", "overlap-gather", "overlap-p2p",
                       "overlap-tree", "overlap-scale", "compressed"})
ONE_STAGE = frozenset({"all_gather"})

_REGISTRY: dict[int, "Communicator"] = {}
_REGISTRY_LOCK = threading.Lock()
_NO_RANGE = contextlib.nullcontext()      # stands in for an NVTX range when LBC_TRACE is off


def _dist():
    dist = import_module("torch.distributed")
    if not dist.is_available() or not dist.is_initialized():
        from ..exceptions import TorchDistributedUnavailableError

        raise TorchDistributedUnavailableError("torch.distributed is not initialized")
    return dist


def get_communicator(group: Any = None, **kwargs) -> "Communicator":
    """Communicator of `group` (default: the world group), created on first use."""

    key = id(group) if group is not None else 0
    with _REGISTRY_LOCK:
        comm = _REGISTRY.get(key)
        if comm is None or comm.closed:
            comm = Communicator(group, **kwargs)
            _REGISTRY[key] = comm
        return comm


def shutdown_communicators() -> None:
    with _REGISTRY_LOCK:
        for comm in _REGISTRY.values():
            comm.close()
        _REGISTRY.clear()


class Communicator:
    def __init__(self, process_group: Any = None, *, arena_bytes: int | None = None, extension_status=None,
                 transport: str = "auto", max_blocks: int = 0) -> None:
        dist = _dist()
        self.process_group = process_group
        self.rank = dist.get_rank(process_group) if process_group is not None else dist.get_rank()
        self.world_size = dist.get_world_size(process_group) if process_group is not None else dist.get_world_size()
        self.arena_bytes = arena_bytes
        self.transport = transport
        self.max_blocks = max_blocks
        self._status = extension_status
        self.peer_group = None
        self.mailbox = None   # PeerMailbox after enable_peer_mailbox()
        self._peer_failed: str | None = None
        self._workspaces: dict[tuple, Any] = {}
        self._subcomms: dict[tuple, Any] = {}
        self.closed = False
        self.stats = {"peer_ops": 0, "torch_ops": 0}

    # -- engines ------------------------------------------------------------
    def _ext(self):
        status = self._status if self._status is not None else load_cuda_extension()
        return status

    def peer_usable(self, tensor: Any, config: CompressionConfig) -> bool:
        if self.transport == "torch" or not bool(getattr(tensor, "is_cuda", False)):
            return False
        if not codec.is_fast_profile(config):
            return False
        status = self._ext()
        if not status.available:
            raise CCDLUnavailableError(
                f"CUDA tensor but the sm_100a extension is not loaded ({status.reason}); refusing to fall back")
        if self._peer_failed is not None:
            if self.transport == "peer":
                raise CCDLUnavailableError(self._peer_failed)
            return False
        return True

    def general_peer_usable(self, tensor: Any, config: CompressionConfig) -> bool:
        """CUDA tensor with a profile the production kernels do not serve (top-k, code-books, stochastic
        rounding): the general kernels plus this library's own peer-memory transport can take it."""

        if self.transport == "torch" or not bool(getattr(tensor, "is_cuda", False)) or codec.is_fast_profile(config):
            return False
        status = self._ext()
        return bool(status.available) and self._peer_failed is None and hasattr(status.module, "quant_general")

    def general_workspace(self, tensor: Any, config: CompressionConfig, dtype: str):
        """Workspace of the general-profile all-reduce able to hold `tensor` (capacity grows in powers of two)."""

        from .fused_general import GeneralPeerWorkspace

        if self.peer_group is not None:
            self.peer_group.check_status()
        key = ("general", dtype, config)
        ws = self._workspaces.get(key)
        if ws is not None and ws.max_numel >= tensor.numel():
            return ws
        cap = 1 << max(16, (max(1, tensor.numel()) - 1).bit_length())
        need = GeneralPeerWorkspace.required_bytes(self.world_size, dtype, config, cap)
        group = self._ensure_peer_group(tensor.device, need)
        if group.bytes_free < need:
            group = self._grow_peer_group(tensor.device, need, f"a {cap}-element general-profile workspace")
        ws = GeneralPeerWorkspace(group, dtype=dtype, config=config, max_numel=cap, max_blocks=self.max_blocks)
        self._workspaces[key] = ws
        return ws

    def _ensure_peer_group(self, device, need_bytes: int):
        from .peer_memory import PeerGroup

        if self.peer_group is None:
            dist = _dist()
            pg = self.process_group if self.process_group is not None else dist.group.WORLD
            # Growing an arena is a collective rebuild (`_grow_peer_group`), so start with room: what the first
            # request needs twice over, and never less than the default (LBC_ARENA_MIB, 1 GiB: small beside
            # 180 GB of HBM, and enough for workspaces of 64 MiB tensors in three dtypes).
            floor = int(float(os.environ.get("LBC_ARENA_MIB", "1024")) * (1 << 20))
            total = int(self.arena_bytes) if self.arena_bytes else max(2 * need_bytes + (64 << 20), floor)
            try:
                self.peer_group = PeerGroup.create(pg, total, device)
            except CCDLUnavailableError as exc:
                self._peer_failed = str(exc)
                raise
        return self.peer_group

    def _grow_peer_group(self, device, need_bytes: int, what: str):
        """The arena has no room for `what`: close it and create a larger one.  Collective over the group, like the
        creation itself; every rank gets here in the same call because tensors of one collective have the same size
        on every rank and the arenas are allocated symmetrically.  The old arena is closed the safe way
        (`PeerGroup.close`: device synchronise, host barrier, then unmap and free); the workspaces that lived in
        it are dropped and come back on their next use, for which the new size leaves room.  A caller-fixed
        `arena_bytes` and an enabled peer mailbox (whose slots and counters live in the arena) rule growth out."""

        old = self.peer_group
        if self.arena_bytes or self.mailbox is not None:
            why = "its size was fixed by arena_bytes" if self.arena_bytes else "a peer mailbox lives in it"
            raise CCDLUnavailableError(
                f"peer arena too small for {what} ({old.bytes_free} < {need_bytes} bytes) and it cannot grow: {why}; "
                "create the communicator with a larger arena_bytes")
        used = old.nbytes - old.bytes_free
        total = max(2 * old.nbytes, used + 2 * need_bytes + (64 << 20))
        old.close()
        self.peer_group = None
        self._workspaces.clear()
        self.stats["arena_rebuilds"] = self.stats.get("arena_rebuilds", 0) + 1
        dist = _dist()
        pg = self.process_group if self.process_group is not None else dist.group.WORLD
        from .peer_memory import PeerGroup

        try:
            self.peer_group = PeerGroup.create(pg, total, device)
        except CCDLUnavailableError as exc:
            self._peer_failed = str(exc)
            raise
        return self.peer_group

    def enable_peer_mailbox(self, capacity_bytes: int, device: Any = None):
        """Collective over the group: reserves one payload slot per source rank in every arena, after which
        `iqsend` / `iqrecv` between any two ranks move their payload with the quantize kernel's own peer
        stores (`PeerMailbox`) instead of an NCCL send/receive pair.  Every rank must call it, in the same
        order relative to other collectives (the arenas are allocated symmetrically)."""

        from .p2p import PeerMailbox

        if self.mailbox is None:
            if device is None:
                import torch

                device = torch.device("cuda", torch.cuda.current_device())
            need = int(capacity_bytes) * self.world_size + (1 << 20)
            group = self._ensure_peer_group(device, need)
            self.mailbox = PeerMailbox(group, capacity_bytes=int(capacity_bytes))
        return self.mailbox

    def workspace(self, tensor: Any, config: CompressionConfig, dtype: str):
        """Fused workspace able to hold `tensor` (capacity grows in powers of two)."""

        from .fused import FusedWorkspace

        if self.peer_group is not None:
            self.peer_group.check_status()       # a kernel of an earlier collective gave up: raise, do not go on
        key = (dtype, config.bit, config.group_size)
        ws = self._workspaces.get(key)
        if ws is not None and ws.max_numel >= tensor.numel():
            return ws
        cap = 1 << max(16, (max(1, tensor.numel()) - 1).bit_length())
        need = FusedWorkspace.required_bytes(self.world_size, dtype, config, cap, True)
        group = self._ensure_peer_group(tensor.device, need)
        if group.bytes_free < need:
            group = self._grow_peer_group(tensor.device, need, f"a {cap}-element workspace")
        ws = FusedWorkspace(group, dtype=dtype, config=config, max_numel=cap, max_blocks=self.max_blocks,
                            with_gather_region=True)
        self._workspaces[key] = ws
        return ws

    def _stream_scope(self, tensor: Any, async_op: bool):
        """(context manager, completion factory) for running on the side stream when async."""

        torch = import_module("torch")
        if not async_op:
            import contextlib

            return contextlib.nullcontext(), None
        from .completion import comm_stream

        side = comm_stream(tensor.device)
        side.wait_stream(torch.cuda.current_stream(tensor.device))
        return torch.cuda.stream(side), side

    def _finish(self, result: Any, side_stream: Any, resources=(), info: ExecutionInfo | None = None) -> Any:
        if side_stream is None:
            return result
        ext = self._ext().module
        work = ext.CompressedWork(result, None, None, list(resources), None,
                                  self.peer_group.status_host if self.peer_group else 0)
        work.record(side_stream.cuda_stream)
        if info is None:
            return work
        from ..core.work import BoundCollectiveWork
        from ..core.info import ExecutionCounters

        return BoundCollectiveWork(work, info, ExecutionCounters())

    # -- all-reduce -----------------------------------------------------------
    def all_reduce(self, tensor: Any, *, config: CompressionConfig, op: str = "mean", strategy: str = "auto",
                   async_op: bool = False, dtype: str = "auto", out: Any = None, residual: Any = None,
                   update_residual: bool = True, ef_mode: str = "reference") -> Any:
        if op not in ("sum", "mean"):
            raise UnsupportedCollective(f"all_reduce:{op}", reason="only op='sum' and op='mean' are implemented")
        name = codec.resolve_dtype(dtype, tensor)
        if strategy == "native_nccl":
            result = make_torch_tensor_all_reduce(group=self.process_group)(tensor if out is None else out.copy_(tensor), op)
            return ImmediateWork(result) if async_op else result
        if strategy == "hierarchical":
            return self.hierarchical_all_reduce(tensor, config=config, op=op, async_op=async_op, dtype=dtype, out=out)
        stages = self._stages(strategy)
        if self.peer_usable(tensor, config):
            try:
                ws = self.workspace(tensor, config, name)
            except CCDLUnavailableError:
                if self.transport == "peer":
                    raise
                ws = None
            if ws is not None:
                scope, side = self._stream_scope(tensor, async_op)
                with scope, tracing.nvtx_range("lbc.all_reduce") if tracing.ENABLED else _NO_RANGE:
                    result = ws.all_reduce(tensor, out, residual=residual, update_residual=update_residual, op=op,
                                           stages=stages, ef_mode=ef_mode)
                self.stats["peer_ops"] += 1
                return self._finish(result, side, resources=(tensor, out, residual))
        if self.general_peer_usable(tensor, config) and tensor.is_contiguous() and (out is None or out.is_contiguous()):
            try:
                gws = self.general_workspace(tensor, config, name)
            except CCDLUnavailableError:
                if self.transport == "peer":
                    raise
                gws = None
            if gws is not None:
                scope, side = self._stream_scope(tensor, async_op)
                # a strategy that names the two-stage algorithm gets it (reduce-scatter, requantize, gather); "auto"
                # and "all_gather" keep the one-stage exchange, and so does stochastic rounding
                two = stages == 2 and not config.stochastic
                with scope:
                    result = gws.all_reduce(tensor, out, residual=residual, update_residual=update_residual, op=op,
                                            stages=2 if two else 1)
                self.stats["peer_ops"] += 1
                return self._finish(result, side, resources=(tensor, out, residual))
        result = self._torch_all_reduce(tensor, config, op, stages, name, out, residual, update_residual)
        self.stats["torch_ops"] += 1
        return ImmediateWork(result) if async_op else result

    def bind_all_reduce(self, *, config: CompressionConfig, op: str = "mean", strategy: str = "auto",
                        dtype: str = "auto"):
        """`f(tensor)` for repeated blocking, in-place all-reduces of tensors of one kind (a compiled plan's hot
        path).  What `all_reduce` settles on every call (profile, extension, stage count, dtype name, workspace
        lookup) is settled on the first call here and again only when a tensor outgrows the workspace; the status
        word is still read before every launch.  Everything the fused kernels do not serve goes to `all_reduce`."""

        if op not in ("sum", "mean"):
            raise UnsupportedCollective(f"all_reduce:{op}", reason="only op='sum' and op='mean' are implemented")
        general = strategy in ("native_nccl", "hierarchical")
        stages = None if general else self._stages(strategy)
        held: list[Any] = [None]

        def call(tensor: Any) -> Any:
            ws = held[0]
            # a held workspace is only good while its arena is this communicator's live one (close() frees it)
            if ws is None or ws.group is not self.peer_group or tensor.numel() > ws.max_numel or not tensor.is_cuda:
                ws = held[0] = None
                if not general and self.peer_usable(tensor, config):
                    try:
                        ws = held[0] = self.workspace(tensor, config, codec.resolve_dtype(dtype, tensor))
                    except CCDLUnavailableError:
                        if self.transport == "peer":
                            raise
                if ws is None:
                    return self.all_reduce(tensor, config=config, op=op, strategy=strategy, dtype=dtype)
            else:
                self.peer_group.check_status()
            result = ws.all_reduce(tensor, None, op=op, stages=stages)
            self.stats["peer_ops"] += 1
            return result

        return call

    def _stages(self, strategy: str) -> int | None:
        if strategy in ("auto", "all_reduce"):
            return None
        if strategy in ONE_STAGE:
            return 1
        if strategy in TWO_STAGE:
            return 2
        raise UnsupportedCollective(f"all_reduce:{strategy}", reason="unknown strategy")

    def _torch_all_reduce(self, tensor, config, op, stages, name, out, residual, update_residual):
        torch = import_module("torch")
        prepared = tensor if residual is None else (tensor.float() + residual.float()).to(tensor.dtype)
        from .fused import default_stages

        stages = stages or default_stages(self.world_size, tensor.numel() * tensor.element_size())
        shape = tuple(tensor.shape)
        gather = make_torch_all_gather(group=self.process_group)
        if stages == 1:
            payload = codec.quantize_tensor(prepared, config, extension_status=self._status)
            buffers = [payload_buffer(p) for p in gather(payload).payloads]
            restored = codec.dequantize_reduce_tensors(buffers, shape, config, dtype=name,
                                                       extension_status=self._status, reduce=op)
        else:
            shard, plan = self._torch_reduce_scatter(prepared, config, op, name)
            payload = codec.quantize_tensor(shard, config, extension_status=self._status)
            parts = [codec.dequantize_tensor(payload_buffer(p), (plan.shard_numel,), config, dtype=name,
                                             extension_status=self._status) for p in gather(payload).payloads]
            restored = torch.cat(parts)[:tensor.numel()].reshape(shape)
        if residual is not None and update_residual:
            codec.update_error_feedback_residual(prepared, restored, residual, extension_status=self._status)
        if out is None:
            tensor.copy_(restored)
            return tensor
        out.copy_(restored.reshape(out.shape))
        return out

    def _torch_reduce_scatter(self, tensor, config, op, name):
        torch = import_module("torch")
        flat = tensor.reshape(-1)
        plan = GroupShardPlan.build(flat.numel(), self.world_size, config.group_size, 8)  # same geometry as the fused path
        padded = torch.nn.functional.pad(flat, (0, plan.padded_numel - flat.numel()))
        chunks = [padded[r * plan.shard_numel:(r + 1) * plan.shard_numel].contiguous() for r in range(self.world_size)]
        sent = [codec.quantize_tensor(c, config, extension_status=self._status) for c in chunks]
        received = make_torch_all_to_all(group=self.process_group)(sent)
        shard = codec.dequantize_reduce_tensors(received, (plan.shard_numel,), config, dtype=name,
                                                extension_status=self._status, reduce=op)
        return shard, plan

    # -- reduce-scatter -------------------------------------------------------
    def reduce_scatter_shard(self, tensor: Any, *, config: CompressionConfig, op: str = "mean",
                             async_op: bool = False, dtype: str = "auto", out: Any = None,
                             residual: Any = None) -> Any:
        """Rank r ends up with the reduced shard r as a `ReducedShard`."""

        if op not in ("sum", "mean"):
            raise UnsupportedCollective(f"reduce_scatter:{op}", reason="only op='sum' and op='mean' are implemented")
        torch = import_module("torch")
        name = codec.resolve_dtype(dtype, tensor)
        shape = tuple(tensor.shape)
        n = tensor.numel()
        est = estimate_quantized_size(n, dtype=name, config=config)
        if self.peer_usable(tensor, config):
            from .fused import geometry

            geo = geometry(n, self.world_size, name, config)
            shard = self._validated_out(out, tensor, geo.shard_numel)
            ws = self.workspace(tensor, config, name)
            scope, side = self._stream_scope(tensor, async_op)
            with scope:
                ws.reduce_scatter(tensor.reshape(-1), shard, residual=residual, op=op)
            self.stats["peer_ops"] += 1
            result = ReducedShard(shard=shard, shard_index=self.rank, shard_numel=geo.shard_numel,
                                  original_shape=shape, original_numel=n, world_size=self.world_size, reduce=op,
                                  padded_numel=geo.shard_numel * self.world_size, dtype=name,
                                  transport="fused_peer_scatter",
                                  metadata={"fused": True, "caller_owned_output": out is not None,
                                            "payload_bytes": est.quantized_bytes, "group_aligned": True})
            return self._finish(result, side, resources=(tensor, shard, residual))
        shard, plan = self._torch_reduce_scatter(tensor, config, op, name)
        if out is not None:
            self._validated_out(out, tensor, plan.shard_numel).copy_(shard)
            shard = out
        self.stats["torch_ops"] += 1
        result = ReducedShard(shard=shard, shard_index=self.rank, shard_numel=plan.shard_numel, original_shape=shape,
                              original_numel=n, world_size=self.world_size, reduce=op,
                              padded_numel=plan.padded_numel, dtype=name, transport="compressed_all_to_all",
                              metadata={"fused": False, "caller_owned_output": out is not None,
                                        "payload_bytes": est.quantized_bytes})
        return ImmediateWork(result) if async_op else result

    @staticmethod
    def _validated_out(out: Any, tensor: Any, shard_numel: int) -> Any:
        """Caller-owned output checks (parity: reduce_scatter_transport.py:390-431)."""

        torch = import_module("torch")
        if out is None:
            return torch.empty(shard_numel, dtype=tensor.dtype, device=tensor.device)
        if hasattr(out, "tensor") and hasattr(out, "mark_submitting"):  # an output lease
            out = out.tensor
        if tuple(out.shape) != (shard_numel,):
            raise ValueError(f"out must have shape ({shard_numel},), got {tuple(out.shape)}")
        if out.dtype != tensor.dtype:
            raise TypeError("out must have the input's dtype")
        if out.device != tensor.device:
            raise ValueError("out must live on the input's device")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
        a0, a1 = tensor.data_ptr(), tensor.data_ptr() + tensor.numel() * tensor.element_size()
        b0, b1 = out.data_ptr(), out.data_ptr() + out.numel() * out.element_size()
        if a0 < b1 and b0 < a1:
            raise ValueError("out must not alias the input")
        return out

    def reduce_scatter_full(self, tensor: Any, *, config: CompressionConfig, op: str = "mean",
                            dtype: str = "auto") -> Any:
        """Reduce-scatter followed by a compressed all-gather of the shards: the full reduced tensor."""

        return self.all_reduce(tensor.clone(), config=config, op=op, strategy="reduce_scatter", dtype=dtype)

    # -- all-gather -------------------------------------------------------------
    def all_gather(self, tensor: Any, *, config: CompressionConfig, async_op: bool = False,
                   dtype: str = "auto") -> Any:
        torch = import_module("torch")
        name = codec.resolve_dtype(dtype, tensor)
        shape = tuple(tensor.shape)
        if self.peer_usable(tensor, config):
            ws = self.workspace(tensor, config, name)
            # rows of one buffer: the decode of all W payloads is then a single launch
            outs = list(torch.empty((self.world_size,) + shape, dtype=tensor.dtype, device=tensor.device).unbind(0))
            scope, side = self._stream_scope(tensor, async_op)
            with scope:
                ws.all_gather(tensor.contiguous(), outs)
            self.stats["peer_ops"] += 1
            return self._finish(outs, side, resources=(tensor,))
        payload = codec.quantize_tensor(tensor, config, extension_status=self._status)
        gathered = make_torch_all_gather(group=self.process_group)(payload)
        outs = [codec.dequantize_tensor(payload_buffer(p), shape, config, dtype=name, extension_status=self._status)
                for p in gathered.payloads]
        self.stats["torch_ops"] += 1
        return ImmediateWork(outs) if async_op else outs

    # -- hierarchical -------------------------------------------------------------
    def sub_communicators(self, local_group_size: int):
        """(local communicator, inter communicator) for contiguous groups of `local_group_size` ranks.

        Group creation is collective: every rank creates every group, in the same order
        (parity: hierarchical_transport.py:178-215, cuda/transports/hierarchical.py:184-265).
        """

        L = int(local_group_size)
        if L <= 0 or self.world_size % L != 0:
            raise UnsupportedCollective("all_reduce:hierarchical",
                                        reason=f"world size {self.world_size} is not a multiple of the local group size {L}")
        key = ("hier", L)
        if key in self._subcomms:
            return self._subcomms[key]
        dist = _dist()
        base = list(range(self.world_size)) if self.process_group is None else dist.get_process_group_ranks(self.process_group)
        from ..core.chunking import hierarchy_groups

        local_groups, inter_groups = hierarchy_groups(base, L)
        local_pg = inter_pg = None
        for node, ranks in enumerate(local_groups):
            pg = dist.new_group(ranks)
            if self.rank // L == node:
                local_pg = pg
        for lane, ranks in enumerate(inter_groups):
            pg = dist.new_group(ranks)
            if self.rank % L == lane:
                inter_pg = pg
        pair = (Communicator(local_pg, extension_status=self._status, transport=self.transport),
                Communicator(inter_pg, extension_status=self._status, transport=self.transport))
        self._subcomms[key] = pair
        return pair

    def hierarchical_all_reduce(self, tensor: Any, *, config: CompressionConfig, op: str = "mean",
                                async_op: bool = False, dtype: str = "auto", out: Any = None,
                                local_group_size: int | None = None) -> Any:
        """Three stages: intra-group compressed reduce-scatter (full -> shard), inter-group
        compressed all-reduce of the shard, intra-group compressed all-gather (shard -> full).

        On CUDA tensors the three stages are chained on one stream over the sub-groups' fused workspaces:
        scatter + reduce kernels leave this rank's shard in a cached dense buffer, the pipelined kernel
        all-reduces it in place across the groups, and one quantize launch plus one decode launch gather the
        group's shards straight into the output (reference: the compiled three-stage chain with one stream
        per stage, ccdl_comm/cuda/transports/hierarchical.py:184-265).
        """

        torch = import_module("torch")
        L = local_group_size or self._default_local_group()
        local, inter = self.sub_communicators(L)
        name = codec.resolve_dtype(dtype, tensor)
        n = tensor.numel()
        target = tensor if out is None else out
        if self.peer_usable(tensor, config) and tensor.is_contiguous() and target.is_contiguous():
            from .fused import geometry

            geo = geometry(n, local.world_size, name, config)
            ws_local = local.workspace(tensor, config, name)
            key = ("hier_shard", name, geo.shard_numel, str(tensor.device))
            shard = self._subcomms.get(key)
            if shard is None:
                shard = self._subcomms[key] = torch.empty(geo.shard_numel, dtype=tensor.dtype, device=tensor.device)
            ws_inter = inter.workspace(shard, config, name) if inter.world_size > 1 else None
            scope, side = self._stream_scope(tensor, async_op)
            with scope:
                ws_local.reduce_scatter(tensor.reshape(-1), shard, op=op)
                if ws_inter is not None:
                    ws_inter.all_reduce(shard, op=op, stages=1)
                ws_local.gather_shards(shard, target.reshape(-1))
            self.stats["peer_ops"] += 1
            return self._finish(target, side, resources=(tensor, target, shard))
        shard = local.reduce_scatter_shard(tensor, config=config, op=op, dtype=name)
        piece = shard.shard
        if inter.world_size > 1:
            piece = inter.all_reduce(piece, config=config, op=op, strategy="all_gather", dtype=name)
        parts = local.all_gather(piece, config=config, dtype=name)
        full = torch.cat([p.reshape(-1) for p in parts])[:n].reshape(tensor.shape)
        target.copy_(full)
        return ImmediateWork(target) if async_op else target

    def _default_local_group(self) -> int:
        import os

        env = os.environ.get("CCDL_LOCAL_GROUP_SIZE") or ""
        if env.isdigit() and int(env) > 0:
            return int(env)
        for cand in (4, 2):
            if self.world_size % cand == 0 and self.world_size > cand:
                return cand
        return self.world_size

    # -- lifecycle ------------------------------------------------------------------
    def check_status(self) -> None:
        if self.peer_group is not None:
            self.peer_group.check_status()

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        for entry in self._subcomms.values():
            if isinstance(entry, tuple):             # (local communicator, inter communicator); other entries are buffers
                for sub in entry:
                    sub.close()
        if self.peer_group is not None:
            self.peer_group.close()
            self.peer_group = None
        self._workspaces.clear()
