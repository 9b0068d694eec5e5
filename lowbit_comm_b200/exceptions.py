"""Error types raised by the library (parity: ccdl_comm/exceptions.py:4-29)."""

from __future__ import annotations


class CCDLError(RuntimeError):
    """Root of every error this library raises on purpose."""


class CCDLUnavailableError(CCDLError):
    """The sm_100a extension, CUDA, or peer memory is not usable here."""


class BackendRegistrationError(CCDLError):
    """A backend factory or executor broke the registry contract."""


class TorchDistributedUnavailableError(CCDLError):
    """`torch.distributed` is missing or not initialised for the request."""


class AsyncCommunicationError(CCDLError):
    """A device-side bounded wait expired or a peer reported a failure.

    `status` carries the decoded device status word (code, peer, slot, epoch
    seen, epoch expected) when one is available.
    """

    def __init__(self, message: str, *, status: dict | None = None) -> None:
        super().__init__(message)
        self.status = dict(status or {})


class UnsupportedCollective(CCDLError):
    """The requested collective/strategy cannot run in this context."""

    def __init__(self, collective: str, *, reason: str | None = None) -> None:
        text = f"unsupported CCDL collective or strategy: {collective}"
        super().__init__(f"{text} ({reason})" if reason else text)
        self.collective = collective
        self.reason = reason
