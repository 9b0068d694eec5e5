"""Errors this library raises on purpose, and the device status word some of them carry.

The class names are the reference's (ccdl_comm/exceptions.py:4-29) so that `except` clauses written against
it keep working.  `AsyncCommunicationError` and `DeviceWaitStatus` belong to the peer-memory kernels: a
bounded wait that gives up writes five integers into pinned host memory, and the next host-side check turns
them into an exception instead of leaving a hung stream.
"""

from __future__ import annotations

from typing import NamedTuple

WAIT_PHASE_NAMES = ("reduce-scatter", "all-gather", "p2p data", "p2p ack")
# phases of the pipelined all-reduce kernel (ops/csrc/pipe_kernels.cu)
PIPE_PHASE_NAMES = {8: "pipelined all-reduce: quantize rows", 9: "pipelined all-reduce: peers' quantized rows",
                    10: "pipelined all-reduce: an owner's reduced rows", 11: "pipelined all-reduce: rendezvous",
                    12: "pipelined all-reduce: a bulk load never completed"}


class DeviceWaitStatus(NamedTuple):
    """What a kernel recorded when a wait on a peer's flag ran out of time.  `code` 0 means nothing
    happened; `peer` is the flag slot (the rank whose signal never arrived)."""

    code: int = 0
    phase: int = 0
    peer: int = 0
    seen: int = 0
    expected: int = 0

    @property
    def timed_out(self) -> bool:
        return self.code != 0

    @property
    def phase_name(self) -> str:
        if self.phase in PIPE_PHASE_NAMES:
            return PIPE_PHASE_NAMES[self.phase]
        return WAIT_PHASE_NAMES[self.phase] if 0 <= self.phase < len(WAIT_PHASE_NAMES) else f"phase {self.phase}"

    def describe(self, rank: int) -> str:
        return (f"device wait timed out on rank {rank} (phase {self.phase}: {self.phase_name}, flag {self.peer}, "
                f"saw epoch {self.seen}, expected {self.expected})")


class CCDLError(RuntimeError):
    """Root of every error this library raises on purpose."""


class CCDLUnavailableError(CCDLError):
    """The sm_100a extension, CUDA, or peer memory is not usable here."""


class TorchDistributedUnavailableError(CCDLError):
    """`torch.distributed` is missing or not initialised for the request."""


class BackendRegistrationError(CCDLError):
    """A backend factory, selector or executor broke the registry contract."""


class UnsupportedCollective(CCDLError):
    """The requested collective/strategy cannot run in this context.  Routes and backends raise it to
    decline a request; the caller then tries its next candidate."""

    def __init__(self, collective: str, *, reason: str | None = None) -> None:
        self.collective, self.reason = collective, reason
        because = f" ({reason})" if reason else ""
        super().__init__(f"unsupported CCDL collective or strategy: {collective}{because}")


class AsyncCommunicationError(CCDLError):
    """A device-side bounded wait expired, or a peer reported a failure.  `status` holds the decoded device
    status (keys `code`, `phase`, `peer`, `seen`, `expected`) when there is one, else it is empty."""

    def __init__(self, message: str, *, status: dict | DeviceWaitStatus | None = None) -> None:
        super().__init__(message)
        if isinstance(status, DeviceWaitStatus):
            status = status._asdict()
        self.status = dict(status or {})

    @classmethod
    def from_wait(cls, rank: int, status: DeviceWaitStatus) -> "AsyncCommunicationError":
        return cls(status.describe(rank), status=status)
