"""Weight-streaming products for steps of few tokens, as parts use them.

A step of up to 64 tokens in bfloat16 is a read of the weights: its products run on this
repository's weight-streaming kernels with the norm in the prologue (where the rows are few and
narrow enough) and SwiGLU or the residual add in the epilogue, instead of library products with
element-wise launches around them.  The functions here choose the kernel form (mma.sync or
tcgen05, norm fused or launched on its own) from the sizes, so that an arrangement and any
feed-forward that offers a few-token path (`FeedForward.forward_few_tokens`) are written once
against three operations:

    normed_linear(h, norm, w, out, ctx)                 out = norm(h) @ w^T
    normed_swiglu(h, norm, gate_up, gate_mult, out, ctx) out = silu(g * gate_mult) * u,  [g | u] = norm(h) @ gate_up^T
    add_products(h, [(x, w, scale), ...], ctx)          h += sum scale * x @ w^T        (one or two products)

h is the float32 residual stream [T, D]; x, w and out are bfloat16.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch

from ..kernels import ops as K
from .base import Norm

Tensor = torch.Tensor

# The tcgen05 form of the products for the larger few-token steps (PMM_TC_SKINNY=0: the mma.sync
# form throughout).
_TC_SKINNY = os.environ.get("PMM_TC_SKINNY", "1") == "1"


def eligible(ctx, width: int) -> bool:
    """Whether a step may take the weight-streaming products for rows of ``width``."""
    return (ctx.dtype == torch.bfloat16 and ctx.n_tokens <= K.SKINNY_MAX_TOKENS and width % 8 == 0
            and K.skinny_fits(ctx.n_tokens, width))


def _prologue(h: Tensor, norm: Norm):
    """(weight, eps) when the norm can run inside the product's prologue for these rows."""
    if h.shape[0] > K.SKINNY_NORM_MAX_TOKENS or h.shape[1] > K.SKINNY_NORM_MAX_WIDTH:
        return None
    return norm.rms_prologue()


def _normed(h: Tensor, norm: Norm, ctx) -> Tensor:
    x = ctx.workspace.alloc(tuple(h.shape), ctx.dtype)
    norm.forward(h, [], x, None, ctx)
    return x


def _tensor_core(T: int) -> bool:
    # beyond 32 tokens the tcgen05 form of the products is the faster one (where it takes the sizes)
    return _TC_SKINNY and T >= K.SKINNY_TC_FROM_TOKENS


def normed_linear(h: Tensor, norm: Norm, w: Tensor, out: Tensor, ctx) -> None:
    pro = _prologue(h, norm)
    if pro is not None:
        K.skinny_linear_norm(h, pro[0], pro[1], w, out)
        return
    x = _normed(h, norm, ctx)
    if _tensor_core(h.shape[0]) and K.skinny_tc_supported("store", x, w, out):
        K.skinny_tc_linear(x, w, out)
    else:
        K.skinny_linear(x, w, out)


def normed_swiglu(h: Tensor, norm: Norm, gate_up: Tensor, gate_mult: float, out: Tensor, ctx) -> None:
    pro = _prologue(h, norm)
    if pro is not None:
        K.skinny_swiglu_norm(h, pro[0], pro[1], gate_up, gate_mult, out)
        return
    x = _normed(h, norm, ctx)
    if _tensor_core(h.shape[0]) and K.skinny_tc_supported("swiglu", x, gate_up, out):
        K.skinny_tc_swiglu(x, gate_up, gate_mult, out)
    else:
        K.skinny_swiglu(x, gate_up, gate_mult, out)


def add_products(h: Tensor, products: Sequence[Tuple[Tensor, Tensor, float]], ctx) -> None:
    products = list(products)
    if _tensor_core(h.shape[0]) and all(K.skinny_tc_supported("residual", x, w) for x, w, _ in products):
        K.skinny_tc_residual(h, products)
    else:
        K.skinny_residual(h, products)
