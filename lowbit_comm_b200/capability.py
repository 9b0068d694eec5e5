"""Import-safe runtime probe.

Parity: ccdl_comm/capability.py:10-166 (`CapabilityReport`, `detect`,
`to_dict`, `to_backend_capabilities`).  The reference still reports
`compressed_collectives=False, ddp_hook=False` from `detect()` although both
exist there; this probe reports what is actually usable and adds the facts a
Blackwell deployment cares about (architecture, peer access, extension build).
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field
from typing import Any

_COLLECTIVES = ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "reduce", "gather",
                "scatter", "barrier", "send", "recv")
_STRATEGIES = ("all_gather", "reduce_scatter", "topology", "hierarchical", "compressed", "native_nccl", "auto")


@dataclass(frozen=True)
class CapabilityReport:
    available: bool
    cuda: bool
    torch_version: str | None = None
    cuda_arch: str | None = None
    quantize: bool = False
    compressed_collectives: bool = False
    ddp_hook: bool = False
    reason: str | None = None
    warnings: tuple[str, ...] = ()
    details: dict = field(default_factory=dict, compare=False)

    @classmethod
    def unavailable(cls, reason: str, **kw: Any) -> "CapabilityReport":
        return cls(available=False, cuda=kw.pop("cuda", False), reason=reason, **kw)

    def to_dict(self) -> dict:
        return {
            "available": self.available,
            "cuda": self.cuda,
            "torch_version": self.torch_version,
            "cuda_arch": self.cuda_arch,
            "ops": {"quantize": self.quantize, "compressed_collectives": self.compressed_collectives,
                    "ddp_hook": self.ddp_hook},
            "reason": self.reason,
            "warnings": list(self.warnings),
        }

    def to_backend_capabilities(self, backend: str = "cuda"):
        from .core.backend import BackendCapabilities

        if not self.available:
            return BackendCapabilities(backend=backend, available=False,
                                       reason=self.reason or "backend is unavailable", warnings=self.warnings)
        features = {"quantize"} if self.quantize else set()
        if self.compressed_collectives:
            features.add("compressed_collectives")
        if self.ddp_hook:
            features.add("ddp_hook")
        if self.details.get("peer_access"):
            features.add("peer_memory")
        return BackendCapabilities(
            backend=backend, available=True, collectives=frozenset(_COLLECTIVES), strategies=frozenset(_STRATEGIES),
            dtypes=frozenset({"fp16", "bf16", "fp32"}), bits=frozenset({4, 8}),
            output_layouts=frozenset({"full", "shard"}), supports_async=True, supports_dynamic_shape=True,
            features=frozenset(features), warnings=self.warnings,
            details={"cuda_arch": self.cuda_arch, "torch_version": self.torch_version, **self.details})


def detect(*, import_torch: Callable[[], Any] | None = None,
           import_extension: Callable[[], Any] | None = None) -> CapabilityReport:
    """Probe torch, CUDA, the device architecture and the sm_100a extension."""

    try:
        torch = import_torch() if import_torch is not None else __import__("torch")
    except Exception as exc:  # noqa: BLE001
        return CapabilityReport.unavailable(f"torch is not importable: {exc}")
    version = str(getattr(torch, "__version__", "unknown"))
    cuda_mod = getattr(torch, "cuda", None)
    has_cuda = bool(cuda_mod is not None and cuda_mod.is_available())
    if not has_cuda:
        return CapabilityReport.unavailable("CUDA is not available to torch", torch_version=version,
                                            ddp_hook=True,
                                            warnings=("only the torch-fallback codec and gloo/CPU paths can run",))
    major, minor = cuda_mod.get_device_capability()
    arch = f"sm_{major}{minor}"
    from .ops.loader import load_cuda_extension

    status = load_cuda_extension(importer=import_extension)
    notes: list[str] = []
    if arch != "sm_100":
        notes.append(f"kernels are built for sm_100a; this device is {arch}")
    if not status.available:
        return CapabilityReport(available=False, cuda=True, torch_version=version, cuda_arch=arch,
                                reason=f"extension unavailable: {status.reason}", warnings=tuple(notes))
    details = {"device_count": cuda_mod.device_count(), "extension_arch": getattr(status.module, "ARCH", None)}
    try:
        cur = cuda_mod.current_device()
        details["peer_access"] = all(status.module.can_access_peer(cur, p) for p in range(cuda_mod.device_count()))
    except Exception as exc:  # noqa: BLE001
        details["peer_access"] = False
        notes.append(f"peer access probe failed: {exc}")
    usable = arch == "sm_100"
    return CapabilityReport(available=usable, cuda=True, torch_version=version, cuda_arch=arch, quantize=usable,
                            compressed_collectives=usable, ddp_hook=True,
                            reason=None if usable else notes[0], warnings=tuple(notes), details=details)
