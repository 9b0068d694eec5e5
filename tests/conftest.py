import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def _cuda_ok() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_ok():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _same_random_numbers_every_run():
    """Tests that draw tensors without a generator of their own get the same numbers on every run, so a
    tolerance that holds once holds always."""

    import torch

    torch.manual_seed(20240229)
    yield


@pytest.fixture(scope="session")
def ext():
    """The sm_100a extension; a GPU box without it is a failure, not a skip."""

    from lowbit_comm_b200.ops.loader import require_extension

    return require_extension()


def spawn_ranks(worker, make_args, nprocs: int, attempts: int = 2) -> None:
    """Run `worker(rank, *make_args(port))` as `nprocs` spawned processes rendezvousing on 127.0.0.1.

    The free port is probed and released before the ranks bind it, so another process can take it in
    between; a failed rendezvous is retried once on a fresh port (a genuine failure fails both times).
    """

    import socket

    import torch.multiprocessing as mp

    last = None
    for _ in range(attempts):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        try:
            mp.start_processes(worker, args=make_args(port), nprocs=nprocs, join=True, start_method="spawn")
            return
        except Exception as exc:  # noqa: BLE001
            last = exc
            text = str(exc)
            if not any(k in text for k in ("Address already in use", "EADDRINUSE", "Connection refused",
                                           "connect() timed out", "failed to connect")):
                raise
    raise last
