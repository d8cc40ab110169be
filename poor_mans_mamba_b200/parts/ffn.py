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
from .base import FeedForward, ParamSpec, register_feed_forward

Tensor = torch.Tensor

# The fused tcgen05 kernel (gate/up projection with the activation in its epilogue) is correct
# and tested but, with 128 x 128 tiles fed by one block, bound by the L2-to-SM operand rate
# (about 360-690 TFLOP/s measured against the library's 960-1460 on the same shapes), so the
# library product plus the activation kernel stays the default until the two-block 256 x 256
# form exists.  PMM_TCGEN05_FFN=1 switches it on for portions of at least this many tokens.
_TC_FROM_TOKENS = 128
_TC_ENABLED = os.environ.get("PMM_TCGEN05_FFN", "0") == "1"


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
        if _TC_ENABLED and T >= _TC_FROM_TOKENS and K.tc_gemm_supported(x, self.gate_up, f, True):
            # prompt portions in bfloat16: gate and up projection with the activation in the
            # epilogue of one tcgen05 kernel; the [T, 2F] intermediate is never written
            K.tc_gemm_swiglu(x, self.gate_up, self.gate_multiplier, act)
        else:
            gu = ctx.workspace.alloc((T, 2 * f), x.dtype)
            K.linear(x, self.gate_up, gu)
            K.silu_mul(gu, self.gate_multiplier, act)
        K.linear(act, self.down, out)


register_feed_forward("swiglu", SwiGLU)
