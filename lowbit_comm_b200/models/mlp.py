"""Synthetic MLP used by the CPU/gloo correctness configuration and the examples.

The reference keeps an equivalent model inside its benchmark script
(tests/distributed/synthetic_ddp_compare.py:20-32).
"""

from __future__ import annotations

import torch
from torch import nn


class SyntheticMLP(nn.Module):
    def __init__(self, widths=(1024, 4096, 4096, 1024), dtype=torch.float32, bias: bool = True) -> None:
        super().__init__()
        layers: list[nn.Module] = []
        for i, (a, b) in enumerate(zip(widths[:-1], widths[1:])):
            layers.append(nn.Linear(a, b, bias=bias, dtype=dtype))
            if i < len(widths) - 2:
                layers.append(nn.GELU())
        self.net = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)
