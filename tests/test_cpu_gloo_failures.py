"""Failure detection with host-side faults only (gloo ranks on CPU, nothing on a GPU).

A rank that leaves between two steps must turn the next collective of the remaining rank into an
exception within the process group's timeout, not into a hang; an asynchronous work object must
cache that exception and raise it again on every later wait.
"""

import datetime
import json
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
from conftest import spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    import lowbit_comm_b200 as lbc

    cfg = lbc.CompressionConfig()
    x = (torch.randn(64 * 50, generator=torch.Generator().manual_seed(rank)) * 0.01).to(torch.bfloat16)
    # step 1: everyone is here
    first = lbc.compressed_all_reduce(x.clone(), config=cfg, strategy="all_gather")
    assert torch.isfinite(first.float()).all()
    if rank == world - 1:
        # this rank leaves between steps: no collective of its own is in flight
        os._exit(0)
    time.sleep(0.5)
    report = {"rank": rank}
    t0 = time.time()
    try:
        lbc.compressed_all_reduce(x.clone(), config=cfg, strategy="all_gather")
        report["outcome"] = "completed"
    except BaseException as exc:  # noqa: BLE001 - the point is that *something* is raised
        report["outcome"] = "raised"
        report["error"] = type(exc).__name__
    report["seconds"] = time.time() - t0
    # the asynchronous form: the error surfaces on wait() and is raised again on a second wait()
    try:
        work = lbc.compressed_all_reduce(x.clone(), config=cfg, strategy="all_gather", async_op=True)
        errors = []
        for _ in range(2):
            try:
                work.wait()
            except BaseException as exc:  # noqa: BLE001
                errors.append(type(exc).__name__)
        report["async_errors"] = errors
    except BaseException as exc:  # noqa: BLE001 - raised at launch instead of at wait
        report["async_errors"] = [type(exc).__name__, type(exc).__name__]
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as fh:
        json.dump(report, fh)
    os._exit(0)   # the process group is broken; do not try to tear it down collectively


@pytest.mark.timeout(180)
def test_a_rank_that_left_turns_the_next_collective_into_an_error(tmp_path):
    world = 2
    spawn_ranks(_worker, lambda port: (world, port, str(tmp_path)), world)
    report = json.load(open(tmp_path / "rank0.json"))
    assert report["outcome"] == "raised", report
    assert report["seconds"] < 60, report
    assert len(report["async_errors"]) == 2 and report["async_errors"][0] == report["async_errors"][1], report
