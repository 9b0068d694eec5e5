"""Makes the unmodified reference (`ccdl_comm`, installed under baseline/_ref)
importable in this process, including its CUDA extension.

Install record: `pip install --no-index --no-build-isolation --no-deps --target
baseline/_ref` of the reference root (an empty meta package), then of
packages/ccdl-core (all Python) and packages/ccdl-cuda with
CCDL_COMM_BUILD_CUDA=1 TORCH_CUDA_ARCH_LIST=10.0 from a copy under /tmp (its
code generators write into the source tree).
"""

from __future__ import annotations

import ctypes
import os
import sys
from pathlib import Path

REF_ROOT = Path(__file__).resolve().parent / "_ref"
SHIM = REF_ROOT / "libthcp_event_shim.so"


def reference_available() -> tuple[bool, str]:
    if not (REF_ROOT / "ccdl_comm" / "__init__.py").exists():
        return False, "baseline/_ref/ccdl_comm is not installed"
    return True, ""


def activate(*, need_cuda_extension: bool = True):
    """Put the reference on sys.path and return (ccdl_comm module, extension status)."""

    ok, why = reference_available()
    if not ok:
        raise ImportError(why)
    import torch  # the extension links against libtorch: load it first

    if SHIM.exists():
        lib = ctypes.CDLL(str(SHIM), mode=os.RTLD_GLOBAL | os.RTLD_NOW)
        slot = ctypes.c_void_p.in_dll(lib, "THCPEventClass")
        base = getattr(torch._C, "_CudaEventBase", None)
        if base is not None and not slot.value:
            slot.value = id(base)  # CPython: id() is the object's address
    if str(REF_ROOT) not in sys.path:
        sys.path.insert(0, str(REF_ROOT))
    import ccdl_comm
    from ccdl_comm.cuda.loader import load_cuda_extension

    status = load_cuda_extension()
    if need_cuda_extension and not status.available:
        raise ImportError(f"reference CUDA extension unavailable: {status.reason}")
    return ccdl_comm, status
