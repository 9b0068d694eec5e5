"""Public tensor-level collectives (parity: ccdl_comm/collectives/__init__.py)."""

from .all_gather import compressed_all_gather
from .all_reduce import compressed_all_reduce
from .hierarchical import compressed_hierarchical_all_reduce
from .native import (all_gather, all_reduce, all_to_all, barrier, broadcast, compile_collective, context_from_tensor,
                     gather, native_collectives, reduce, reduce_scatter, scatter)
from .reduce_scatter import compressed_reduce_scatter, compressed_reduce_scatter_shard


def __getattr__(name):
    if name in ("compressed_all_gather_dynamic", "qall_gather_dyn", "compile_dynamic_all_gather"):
        from . import dynamic_all_gather

        return getattr(dynamic_all_gather, name)
    raise AttributeError(name)
