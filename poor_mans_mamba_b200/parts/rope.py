"""Rotate-half rotary position encoding.

inv_freq[i] = 1 / theta^(2i/Dh) for i < Dh/2, made in float32 exactly as the reference
does (src/ops/cpu_backend.cpp:14-21: ``1.f / pow(theta, float(2i)/float(Dh))`` with theta
a float32); the angle pos*inv_freq and its sine and cosine are float32 in the kernel.
The whole head is rotated; there is no scaling of positions.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, register_position_encoding

Tensor = torch.Tensor


class RotaryEncoding(PositionEncoding):
    """Fused into the attention mixer's query/key preparation kernel through ``inv_freq``."""

    def __init__(self, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError("rotary encoding needs an even head size")
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.inv_freq: Optional[Tensor] = None

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        i = torch.arange(self.head_dim // 2, dtype=torch.float32)
        theta32 = torch.tensor(self.theta, dtype=torch.float32)
        inv = 1.0 / torch.pow(theta32, (2.0 * i) / float(self.head_dim))
        self.inv_freq = inv.to(device=device, dtype=torch.float32).contiguous()


class NoPositionEncoding(PositionEncoding):
    """Queries and keys are used as projected."""
    inv_freq = None

    def __init__(self, head_dim: int = 0):
        self.head_dim = int(head_dim)


register_position_encoding("rotary", RotaryEncoding)
register_position_encoding("none", NoPositionEncoding)
