"""Import-safe access to the native extension.

Parity: ccdl_comm/cuda/loader.py:9-43 — `load_cuda_extension()` reports a status
object instead of raising, so that CPU-only hosts can import the package.
`require_extension()` is the loud variant used by every GPU code path: on a
machine with a GPU a missing extension is an error, never a silent fallback.
"""

from __future__ import annotations

import importlib.util
import threading
from dataclasses import dataclass
from typing import Any

from ..exceptions import CCDLUnavailableError

_LOCK = threading.Lock()
_CACHED: "CudaExtensionStatus | None" = None


@dataclass(frozen=True)
class CudaExtensionStatus:
    available: bool
    module: Any | None = None
    reason: str | None = None


def _import_built() -> Any:
    from .build import EXT_NAME, extension_path

    path = extension_path()
    if not path.exists():
        raise ImportError(f"{path.name} has not been built (run `python -m lowbit_comm_b200.ops.build`)")
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(EXT_NAME, str(path))
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot create an import spec for {path}")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def load_cuda_extension(*, importer=None, refresh: bool = False) -> CudaExtensionStatus:
    """Load `_lbc_cuda` once; never raises."""

    global _CACHED
    if importer is not None:  # injected importer: no caching (used by tests)
        try:
            return CudaExtensionStatus(True, importer(), None)
        except Exception as exc:  # noqa: BLE001
            return CudaExtensionStatus(False, None, f"{type(exc).__name__}: {exc}")
    with _LOCK:
        if _CACHED is None or refresh:
            try:
                _CACHED = CudaExtensionStatus(True, _import_built(), None)
            except Exception as exc:  # noqa: BLE001
                _CACHED = CudaExtensionStatus(False, None, f"{type(exc).__name__}: {exc}")
        return _CACHED


def require_extension(status: CudaExtensionStatus | None = None) -> Any:
    """Return the extension module or raise `CCDLUnavailableError`."""

    active = status if status is not None else load_cuda_extension()
    if not active.available or active.module is None:
        raise CCDLUnavailableError(f"lowbit_comm_b200 sm_100a extension is unavailable: {active.reason}")
    return active.module
