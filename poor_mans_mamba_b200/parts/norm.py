"""RMSNorm with the residual additions folded in.

y = x * (1/sqrt(mean(x^2) + eps)) * w; eps inside the root, the weight multiplies after
normalisation (reference src/ops/cpu/rms_norm.cpp:11-16).  Statistics are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from .base import Norm, ParamSpec, register_norm

Tensor = torch.Tensor


def fold_branches(h: Tensor, pending) -> None:
    """h <- h + sum(scale_i * branch_i), two branches per launch."""
    items = list(pending)
    while items:
        K.add_rmsnorm(h, items[:2], None, 0.0, None)
        items = items[2:]


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float):
        self.width = int(width)
        self.eps = float(eps)
        self.weight: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.width,), kind="vector", init=("ones",))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.weight = params["weight"]

    def rms_prologue(self):
        return self.weight, self.eps

    def forward(self, h: Tensor, pending, out: Tensor, rows: Optional[Tensor], ctx) -> None:
        items = list(pending)
        while len(items) > 2:  # more than two branches: fold the surplus first
            if rows is not None:
                raise ValueError("row-selected norm takes at most two pending branches")
            K.add_rmsnorm(h, items[:2], None, 0.0, None)
            items = items[2:]
        K.add_rmsnorm(h, items, self.weight, self.eps, out, rows)


register_norm("rmsnorm", RMSNorm)
