"""Real multi-GPU runs of the fused collectives and the DDP hook (one process per GPU).

Skipped on a single-GPU box: kernels of different ranks that wait on one another
must never share a GPU.  NVLS is switched off in NCCL; the fused kernels use plain peer loads and
stores except in the multicast-arena test, whose ranks leave only after all of them have drained.
"""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count() -> int:
    import torch

    return torch.cuda.device_count()


def _launch(case: str, world: int, multicast: bool = False) -> str:
    # Short device waits: should one rank fail, the kernels of the others give up in seconds, not minutes.
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, LBC_WAIT_TIMEOUT_MS="20000")
    if multicast:
        # short device waits: if one rank fails, the others drain in seconds and nobody unmaps early
        env.update(LBC_MULTICAST="1", LBC_WAIT_TIMEOUT_MS="3000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29400 + world + (7 if case == "ddp" else 0) + (20 if multicast else 0)),
           os.path.join(ROOT, "tests", "multirank_worker.py"), case]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    tail = (proc.stdout + proc.stderr)[-4000:]
    assert proc.returncode == 0 and f"MULTIRANK-OK {case}" in proc.stdout, tail
    return proc.stdout


@pytest.mark.parametrize("case", ["collectives", "ddp"])
def test_multirank(case):
    count = _gpu_count()
    if count < 2:
        pytest.skip("needs at least two GPUs")
    _launch(case, min(count, 8) if count in (2, 4, 8) else 2)


def test_multirank_multicast_arena():
    """Same collectives with the arenas bound to an NVLink multicast object: broadcasts leave the GPU
    once (`multimem.st`).  Where the multicast arena cannot be set up the library falls back to CUDA
    IPC arenas on every rank, and the run still has to be bit-exact."""

    count = _gpu_count()
    if count < 2:
        pytest.skip("needs at least two GPUs")
    out = _launch("collectives", min(count, 8) if count in (2, 4, 8) else 2, multicast=True)
    assert "multicast=" in out
