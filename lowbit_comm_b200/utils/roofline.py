"""Roofline model of the fused compressed collectives.

T_roof = max(T_hbm, T_link): HBM traffic of the kernels at the measured copy
bandwidth versus compressed bytes that must cross NVLink at the measured
per-direction link bandwidth (770 GB/s on this pool; 900 nominal).
"""

from __future__ import annotations

import json
import os

MEASURED_LINK_GBS = 770.0
FALLBACK_HBM_GBS = 6650.0


def measured_hbm_gbs(repo_root: str | None = None) -> tuple[float, str]:
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def payload_factor(group_size: int = 64, bit: int = 8, element_bytes: int = 2) -> float:
    return (group_size * bit / 8 + element_bytes) / (group_size * element_bytes)


def fused_all_reduce_roofline(nbytes: int, world: int, *, stages: int, error_feedback: bool = True,
                              hbm_gbs: float | None = None, link_gbs: float = MEASURED_LINK_GBS,
                              factor: float | None = None) -> dict:
    c = payload_factor() if factor is None else factor
    hbm_gbs = hbm_gbs or measured_hbm_gbs()[0]
    payload = c * nbytes
    passes = 3 if error_feedback else 1      # grad (+ residual read, prepared write) / result (+ prepared, residual)
    if stages == 2:
        hbm = passes * nbytes + payload + 2 * payload + payload + passes * nbytes
        link = 2 * payload * (world - 1) / world
    else:
        hbm = passes * nbytes + world * payload + world * payload + passes * nbytes
        link = payload * (world - 1)
    t_hbm, t_link = hbm / (hbm_gbs * 1e9), link / (link_gbs * 1e9)
    return {"hbm_bytes": hbm, "link_bytes": link, "t_hbm_us": t_hbm * 1e6, "t_link_us": t_link * 1e6,
            "roofline_us": max(t_hbm, t_link) * 1e6, "bound": "hbm" if t_hbm >= t_link else "nvlink"}
