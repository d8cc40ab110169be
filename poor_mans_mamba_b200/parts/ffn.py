"""Dense SwiGLU feed-forward.

g = (x Wg^T) * gate_multiplier; u = x Wu^T; out = (silu(g) * u) Wd^T; the down
multiplier is the part's ``out_scale`` and is applied where the branch joins the
residual stream (reference src/ops/cpu_backend.cpp:494-531).  Gate and up weights are
stacked into one [2F, D] matrix at load so the two projections are one product.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import streaming
from .base import FeedForward, ParamSpec, register_feed_forward

Tensor = torch.Tensor

# Gate/up projection with the activation in the epilogue of one tcgen05 kernel (256 x 256 tiles,
# TMA operands, accumulators in tensor memory): the [T, 2F] intermediate is never written.
# Measured against the library product plus the activation kernel: 21.6 vs 34.7 us at 2,048 x
# 1,024 -> 2 x 2,048 (launch-bound timing; 19-20 us each inside a step graph), 71 vs 72 us at
# 8,192 tokens, 239 vs 236 us at 2,048 x 3,072 -> 2 x 12,288 (1,290 TFLOP/s).  It runs one tile
# per block in a single wave, so it is used from about 96 tiles on; below that the library's
# smaller tiles fill the GPU better.  PMM_TCGEN05_FFN=0 switches it off.
_TC_FROM_TILES = 96
_TC_ENABLED = os.environ.get("PMM_TCGEN05_FFN", "1") == "1"


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, gate_multiplier: float = 1.0,
                 down_multiplier: float = 1.0):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.gate_multiplier = float(gate_multiplier)
        self.out_scale = float(down_multiplier)
        self.gate_up: Optional[Tensor] = None
        self.down: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        f, d = self.intermediate_size, self.hidden_size
        return [ParamSpec("gate_proj.weight", (f, d)), ParamSpec("up_proj.weight", (f, d)),
                ParamSpec("down_proj.weight", (d, f))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.gate_up = torch.cat([params["gate_proj.weight"], params["up_proj.weight"]], dim=0).contiguous()
        self.down = params["down_proj.weight"].contiguous()

    def forward(self, x: Tensor, ctx, out: Tensor) -> None:
        T = x.shape[0]
        f = self.intermediate_size
        act = ctx.workspace.alloc((T, f), x.dtype)
        tiles = ((T + 255) // 256) * (f // 128)
        if _TC_ENABLED and tiles >= _TC_FROM_TILES and K.tc_gemm_supported(x, self.gate_up, f, True):
            K.tc_gemm_swiglu(x, self.gate_up, self.gate_multiplier, act)
        else:
            gu = ctx.workspace.alloc((T, 2 * f), x.dtype)
            K.linear(x, self.gate_up, gu)
            K.silu_mul(gu, self.gate_multiplier, act)
        K.linear(act, self.down, out)

    def forward_few_tokens(self, h: Tensor, norm, ctx) -> bool:
        """h += down_multiplier * (silu(g) * u) Wd^T with [g | u] = norm(h) [Wg; Wu]^T in two
        weight-streaming launches."""
        if not streaming.eligible(ctx, self.hidden_size):
            return False
        act = ctx.workspace.alloc((h.shape[0], self.intermediate_size), ctx.dtype)
        streaming.normed_swiglu(h, norm, self.gate_up, self.gate_multiplier, act, ctx)
        streaming.add_products(h, [(act, self.down, self.out_scale)], ctx)
        return True

    def streamed_weights(self) -> List[Tensor]:
        return [self.gate_up, self.down]


register_feed_forward("swiglu", SwiGLU)
