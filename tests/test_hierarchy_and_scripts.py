"""Two-level grouping without hardware (8 ranks as 2 x 4, every rank's view), and contract checks on
the benchmark scripts' pure helpers (flags and formulas stay stable without running a GPU)."""

import importlib.util
import os
import sys

import pytest

from lowbit_comm_b200.core.chunking import GroupShardPlan, hierarchy_groups

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("rank", range(8))
def test_two_by_four_membership_from_every_rank(rank):
    local, inter = hierarchy_groups(list(range(8)), 4)
    assert local == [[0, 1, 2, 3], [4, 5, 6, 7]] and inter == [[0, 4], [1, 5], [2, 6], [3, 7]]
    mine_local, mine_inter = local[rank // 4], inter[rank % 4]
    assert rank in mine_local and rank in mine_inter
    assert mine_local.index(rank) == rank % 4 and mine_inter.index(rank) == rank // 4   # group-local ranks
    assert len(mine_local) == 4 and len(mine_inter) == 2                              # 4 -> 2 -> 4
    # full -> shard (1/4 of the tensor) -> inter all-reduce of that shard -> full: the shard every member of
    # an inter group holds is the same slice, so their all-reduce is well defined
    plan = GroupShardPlan.build(1_000_003, 4, 64)
    lo = (rank % 4) * plan.shard_numel
    for peer in mine_inter:
        assert (peer % 4) * plan.shard_numel == lo


def test_grouping_follows_the_order_of_the_given_ranks_and_rejects_ragged_splits():
    local, inter = hierarchy_groups([8, 9, 10, 11, 12, 13], 3)       # a sub-group with global ranks 8..13
    assert local == [[8, 9, 10], [11, 12, 13]] and inter == [[8, 11], [9, 12], [10, 13]]
    with pytest.raises(ValueError):
        hierarchy_groups(list(range(6)), 4)
    with pytest.raises(ValueError):
        hierarchy_groups([], 2)


def test_sweep_roofline_formula():
    # one roofline function for the library and its benchmarks: the sweep script states none of its own
    from lowbit_comm_b200.utils.roofline import fused_all_reduce_roofline

    assert "def roofline_us" not in open(os.path.join(ROOT, "benchmarks", "allreduce_sweep.py")).read()
    nbytes = 256 << 20
    two = fused_all_reduce_roofline(nbytes, 8, stages=2, error_feedback=True, hbm_gbs=6552.3)
    one = fused_all_reduce_roofline(nbytes, 8, stages=1, error_feedback=True, hbm_gbs=6552.3)
    payload = nbytes * 66 / 128
    assert two["t_link_us"] == pytest.approx(2 * payload * 7 / 8 / 770e9 * 1e6)
    assert one["t_link_us"] == pytest.approx(payload * 7 / 770e9 * 1e6)
    assert two["roofline_us"] == max(two["t_hbm_us"], two["t_link_us"]) and one["t_link_us"] > two["t_link_us"]
    # two-stage HBM bytes: 2 x (tensor x 3 + payload) for K1 and K3, 2 payloads for K2
    assert two["t_hbm_us"] == pytest.approx((6 * nbytes + 4 * payload) / 6552.3e9 * 1e6)


def test_bench_contract_flags_and_defaults(monkeypatch):
    bench = _load("bench.py", "bench_script")
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert (args.gpus, args.impl, args.model) == (1, "ours", "gpt2-small") and args.warmup >= 3 and args.steps > 0
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "8", "--steps", "7", "--warmup", "4", "--impl", "reference"])
    args = bench.parse_args()
    assert (args.gpus, args.steps, args.warmup, args.impl) == (8, 7, 4, "reference")
    src = open(os.path.join(ROOT, "bench.py")).read()
    for key in ('"metric"', '"value"', '"unit"', '"n_gpus"', '"ms_per_step"', '"higher_is_better"', '"scaling"',
                '"vs_baseline"', '"dtype"', '"data"', '"config"', '"e2e"', '"h2d_bytes_per_step"',
                '"d2h_bytes_per_step"', '"gpu_launches"', '"clocks"'):
        assert key in src, key


def test_benchmark_and_example_scripts_load_and_describe_their_workload():
    mlp = _load("benchmarks/mlp_ddp.py", "mlp_ddp_script")
    assert mlp.WIDTHS == (2048, 4096, 4096, 4096, 4096, 1024)
    weights = sum(a * b for a, b in zip(mlp.WIDTHS[:-1], mlp.WIDTHS[1:]))
    assert weights == 62_914_560                       # the parameter count of the reference's published run (no biases)
    from lowbit_comm_b200.models.mlp import SyntheticMLP

    tiny = SyntheticMLP((4, 8, 2), bias=False)
    assert sum(p.numel() for p in tiny.parameters()) == 4 * 8 + 8 * 2
    src = open(os.path.join(ROOT, "benchmarks", "mlp_ddp.py")).read()
    for key in ('"metric"', '"value"', '"unit"', '"n_gpus"', '"ms_per_step"', '"h2d_bytes_per_step"', '"gpu_launches"'):
        assert key in src, key
    micro = open(os.path.join(ROOT, "benchmarks", "micro_suite.py")).read()
    for case in ("reduced_shard", "async_vs_sync", "dynamic_gather", "p2p"):
        assert f'case="{case}"' in micro, case
    assert callable(_load("benchmarks/micro_suite.py", "micro_suite_script").main)
    example = _load("examples/cpu_gloo_mlp.py", "cpu_gloo_mlp_example")
    assert example.MODES == ("plain", "wire_codec", "fallback_codec") and callable(example.worker)


@pytest.mark.timeout(600)
def test_benchmark_scripts_dry_run_on_two_cpu_ranks(tmp_path):
    """`--cpu` runs the same calls on gloo ranks: the scripts' use of the public API stays checked without a GPU."""

    import json
    import socket
    import subprocess

    def torchrun(script, *flags):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, script), "--cpu", *flags]
        done = subprocess.run(cmd, capture_output=True, text=True, timeout=500, cwd=ROOT)
        assert done.returncode == 0, done.stderr[-2000:]
        return [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]

    out = tmp_path / "micro.json"
    rows = torchrun("benchmarks/micro_suite.py", "--sizes-mib", "0.25", "--iters", "1", "--warmup", "1", "--out", str(out))
    assert {r["case"] for r in rows} == {"reduced_shard", "async_vs_sync", "dynamic_gather", "p2p"}
    assert all(r["rel_l2"] < 0.01 for r in rows if "rel_l2" in r)
    assert [r["case"] for r in json.loads(out.read_text())] == [r["case"] for r in rows]
    out = tmp_path / "mlp.json"
    (line,) = torchrun("benchmarks/mlp_ddp.py", "--steps", "2", "--warmup", "1", "--repeats", "2", "--out", str(out))
    assert line["unit"] == "samples/s" and line["n_gpus"] == 2 and line["value"] > 0 and line["impl"] == "ours"
    assert len(line["ms_per_step_samples"]) == 2 and line["ms_per_step"] == pytest.approx(
        sum(line["ms_per_step_samples"]) / 2, rel=1e-3)                      # the median of two is their mean
    (line,) = torchrun("benchmarks/mlp_ddp.py", "--impl", "fsdp", "--steps", "1", "--warmup", "1")
    assert line == {"impl": "fsdp", "unavailable": "the FSDP baseline arm runs on CUDA ranks only"}
