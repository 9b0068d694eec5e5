"""Public tensor-level collectives (parity: ccdl_comm/collectives/__init__.py)."""

from .all_gather import compressed_all_gather
from .all_reduce import compressed_all_reduce
from .hierarchical import compressed_hierarchical_all_reduce
from .reduce_scatter import compressed_reduce_scatter, compressed_reduce_scatter_shard

# last: importing the submodules above binds their names (all_gather, all_reduce, reduce_scatter) in this
# package; the pass-through functions of the same names must win
from .native import (all_gather, all_reduce, all_to_all, barrier, broadcast, compile_collective, context_from_tensor,  # noqa: E402,I001
                     gather, native_collectives, reduce, reduce_scatter, scatter)


def __getattr__(name):
    if name in ("compressed_all_gather_dynamic", "qall_gather_dyn", "compile_dynamic_all_gather"):
        from . import dynamic_all_gather

        return getattr(dynamic_all_gather, name)
    raise AttributeError(name)
