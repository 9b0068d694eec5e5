"""Like-for-like performance gates over benchmark result records.

Parity: tests/benchmarks/assert_performance_gate.py:20-99 (baseline vs candidate
matched on identical dimensions, `max_regression=0.02`) and
fused_reduced_shard_gate.py:69-157 (repeat-count, launch-count and
zero-allocation checks).  Added: a roofline gate (fraction of the fused path's
roofline for buckets of at least a given size).
"""

from __future__ import annotations

from dataclasses import dataclass

MATCH_KEYS = ("gpu_name", "world_size", "dtype", "numel", "strategy")


@dataclass(frozen=True)
class GateFinding:
    key: tuple
    baseline_ms: float
    candidate_ms: float
    regression: float
    passed: bool


def _key(record: dict) -> tuple:
    return tuple(record[k] for k in MATCH_KEYS)


def compare_results(baseline: list[dict], candidate: list[dict], *, max_regression: float = 0.02) -> list[GateFinding]:
    """Every candidate row with a matching baseline row must not be slower by more than `max_regression`."""

    base = {_key(r): r for r in baseline}
    findings = []
    for row in candidate:
        ref = base.get(_key(row))
        if ref is None:
            continue
        regression = row["latency_ms"] / ref["latency_ms"] - 1.0
        findings.append(GateFinding(_key(row), ref["latency_ms"], row["latency_ms"], regression,
                                    regression <= max_regression))
    if not findings:
        raise ValueError("no candidate row matches a baseline row on " + ", ".join(MATCH_KEYS))
    return findings


def assert_performance_gate(baseline: list[dict], candidate: list[dict], *, max_regression: float = 0.02) -> None:
    bad = [f for f in compare_results(baseline, candidate, max_regression=max_regression) if not f.passed]
    if bad:
        lines = [f"{f.key}: {f.baseline_ms:.4f} -> {f.candidate_ms:.4f} ms (+{100 * f.regression:.1f} %)" for f in bad]
        raise AssertionError("performance regression beyond the gate:\n" + "\n".join(lines))


def evaluate_fused_gate(runs: list[dict], *, min_repeats: int = 5, launches_per_rank: int | None = None,
                        accuracy_limit: float = 0.02) -> dict:
    """Gate over repeated runs of one case: distinct run ids, launch count, no steady-state allocation, accuracy."""

    ids = {r.get("run_id") for r in runs}
    problems = []
    if len(ids) < min_repeats:
        problems.append(f"only {len(ids)} distinct run ids, need {min_repeats}")
    if launches_per_rank is not None and any(r.get("fused_launches_per_rank") != launches_per_rank for r in runs):
        problems.append(f"expected exactly {launches_per_rank} fused launch(es) per rank")
    if any(r.get("steady_state_allocated_bytes", 0) != 0 for r in runs):
        problems.append("steady-state allocation is not zero")
    if any(r.get("relative_l2", 0.0) > accuracy_limit for r in runs):
        problems.append(f"relative L2 above {accuracy_limit}")
    return {"passed": not problems, "problems": problems, "runs": len(runs)}


def roofline_gate(rows: list[dict], *, min_bytes: int = 64 << 20, min_fraction: float = 0.60) -> list[dict]:
    """Rows (from the sweep) of at least `min_bytes` whose roofline fraction is below `min_fraction`."""

    return [r for r in rows if r.get("roofline_frac") is not None and r.get("mib", 0) * (1 << 20) >= min_bytes
            and r["roofline_frac"] < min_fraction]
