"""Arrangements: how the parts of one layer are ordered around the residual stream.

``ParallelPreNormBlock``: one norm feeds every mixer of the layer; their scaled outputs
join the residual stream in order; then a second norm feeds the feed-forward
(reference src/runtime/runner/falconh1_runner.cpp:20-127: h = (h + mamba) + attn;
h += mlp(norm(h))).  With one mixer it is the usual pre-norm decoder layer; without a
feed-forward it is a bare mixer layer.

The residual stream is float32.  Branch outputs are not added by a kernel of their own:
they stay *pending* on the stream and are folded in by the next norm, which reads and
writes the stream once.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops as K
from .base import (FeedForward, LayerCache, LayerSpec, Mixer, Norm, ParamSpec, Part, StateSpec,
                   build_part, register_arrangement)
from .norm import fold_branches

Tensor = torch.Tensor


# The products after the mixers as ONE launch with barriers over the grid (K.skinny_chain).  Off by
# default: measured at 8 tokens a barrier costs about 3.5 us (fence, arrival, poll), a launch with
# programmatic dependent launch about 1.2 us, so the chain takes 17.8 us where the three separate
# launches take 10.7 us.
_CHAINED = os.environ.get("PMM_SKINNY_CHAIN", "0") == "1"
# The mixers of a layer on parallel streams in steps of many tokens too (PMM_PARALLEL_MIXERS=0: one
# after the other).
_PARALLEL_MIXERS = os.environ.get("PMM_PARALLEL_MIXERS", "1") == "1"
# The tcgen05 form of the weight-streaming products for the larger few-token steps (PMM_TC_SKINNY=0:
# the mma.sync form throughout).
_TC_SKINNY = os.environ.get("PMM_TC_SKINNY", "1") == "1"


class ResidualStream:
    """The float32 hidden state [T, D] of a step plus the branches waiting to be added."""

    def __init__(self, h: Tensor, ctx, n_branch_buffers: int):
        self.h = h
        self.ctx = ctx
        self.pending: List[Tuple[Tensor, float]] = []
        self._buffers = [ctx.workspace.alloc(tuple(h.shape), ctx.dtype) for _ in range(n_branch_buffers)]
        self._taken = 0

    def take_branch(self) -> Tensor:
        """A [T, D] buffer in the storage type for a part to write its output into."""
        if self._taken >= len(self._buffers):
            raise RuntimeError("more branches in flight than the stream has buffers for")
        buf = self._buffers[self._taken]
        self._taken += 1
        return buf

    def add(self, branch: Tensor, scale: float) -> None:
        self.pending.append((branch, float(scale)))

    def normed(self, norm: Norm, rows: Optional[Tensor] = None) -> Tensor:
        """Fold the pending branches into the stream and return norm(stream) (of the selected
        rows only, if given: then the stream itself is left unchanged)."""
        n_rows = self.h.shape[0] if rows is None else rows.numel()
        out = self.ctx.workspace.alloc((n_rows, self.h.shape[1]), self.ctx.dtype)
        norm.forward(self.h, self.pending, out, rows, self.ctx)
        if rows is None:
            self.pending = []
            self._taken = 0
        return out

    def flush(self) -> Tensor:
        fold_branches(self.h, self.pending)
        self.pending = []
        self._taken = 0
        return self.h


class ParallelPreNormBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.prefix = spec.prefix
        self.hidden_size = hidden_size
        self.mixer_norm: Norm = build_part("norm", spec.mixer_norm, width=hidden_size)
        self.mixers: List[Mixer] = [build_part("mixer", m, hidden_size=hidden_size) for m in spec.mixers]
        self.ffn_norm: Optional[Norm] = None
        self.ffn: Optional[FeedForward] = None
        if spec.ffn is not None:
            if spec.ffn_norm is None:
                raise ValueError("a feed-forward needs its norm")
            self.ffn_norm = build_part("norm", spec.ffn_norm, width=hidden_size)
            self.ffn = build_part("feed_forward", spec.ffn, hidden_size=hidden_size)
        self._fused_in: Optional[Tensor] = None
        self._fused_cols: List[Tuple[int, int]] = []

    def parts(self) -> List[Part]:
        out: List[Part] = [self.mixer_norm, *self.mixers]
        if self.ffn is not None:
            out += [self.ffn_norm, self.ffn]
        return out

    def branch_buffers_needed(self) -> int:
        return max(len(self.mixers), 1)

    def state_specs(self) -> List[Tuple[str, StateSpec]]:
        """(qualified name, spec) for every state of every mixer of this layer."""
        return [(f"{m.name}.{s.name}", s) for m in self.mixers for s in m.state_specs()]

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        for p in self.parts():
            p.finalize(dtype, device)
        # One input projection for all mixers that expose theirs.
        if len(self.mixers) > 1 and all(m.input_rows() > 0 for m in self.mixers):
            fused = torch.cat([m.input_weight() for m in self.mixers], dim=0).contiguous()
            start = 0
            for m in self.mixers:
                rows = m.input_rows()
                m.adopt_input_weight(fused[start:start + rows])
                self._fused_cols.append((start, start + rows))
                start += rows
            self._fused_in = fused

    def _few_tokens_path(self, ctx) -> bool:
        """Steps of few tokens in bfloat16 are reads of the weights: they take the fused
        weight-streaming products (norm in the prologue, SwiGLU or the residual add in the
        epilogue) instead of library products with separate element-wise launches."""
        from .ffn import SwiGLU
        from .norm import RMSNorm
        if (ctx.dtype != torch.bfloat16 or ctx.n_tokens > K.SKINNY_MAX_TOKENS or self.hidden_size % 8
                or not K.skinny_fits(ctx.n_tokens, self.hidden_size)):
            return False
        if self._fused_in is None or not isinstance(self.mixer_norm, RMSNorm):
            return False
        if any(m.output_weight() is None or m.output_bias() is not None for m in self.mixers):
            return False
        if len(self.mixers) > 2:
            return False
        if self.ffn is not None and not (isinstance(self.ffn, SwiGLU) and isinstance(self.ffn_norm, RMSNorm)):
            return False
        return True

    _SIDE_STREAMS: Dict[torch.device, "torch.cuda.Stream"] = {}

    @classmethod
    def _side_stream(cls, device: torch.device) -> "torch.cuda.Stream":
        st = cls._SIDE_STREAMS.get(device)
        if st is None:
            st = torch.cuda.Stream(device=device)
            cls._SIDE_STREAMS[device] = st
        return st

    def streamed_weights(self) -> List[Tensor]:
        """The matrices a step of few tokens reads once: what the layer before this one may
        ask the memory system to fetch ahead."""
        ws = [self._fused_in] + [m.output_weight() for m in self.mixers]
        if self.ffn is not None:
            ws += [getattr(self.ffn, "gate_up", None), getattr(self.ffn, "down", None)]
        return [w for w in ws if w is not None]

    def _forward_few_tokens(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        ws = ctx.workspace
        mark = ws.mark()
        h = stream.flush()
        T = h.shape[0]
        side = self._side_stream(h.device) if len(self.mixers) > 1 else None
        main = torch.cuda.current_stream(h.device)
        ahead = getattr(ctx, "fetch_ahead", None)  # the next layer's weights, set by the model
        if ahead and side is None:
            K.l2_prefetch(ahead)
        proj = ws.alloc((T, self._fused_in.shape[0]), ctx.dtype)
        fused_norm = T <= K.SKINNY_NORM_MAX_TOKENS and self.hidden_size <= K.SKINNY_NORM_MAX_WIDTH
        # beyond 32 tokens the tcgen05 form of the products is the faster one (where it takes the sizes)
        tensor_core = _TC_SKINNY and T >= K.SKINNY_TC_FROM_TOKENS
        if fused_norm:
            K.skinny_linear_norm(h, self.mixer_norm.weight, self.mixer_norm.eps, self._fused_in, proj)
        else:
            x = ws.alloc((T, self.hidden_size), ctx.dtype)
            K.add_rmsnorm(h, [], self.mixer_norm.weight, self.mixer_norm.eps, x)
            if tensor_core and K.skinny_tc_supported("store", x, self._fused_in, proj):
                K.skinny_tc_linear(x, self._fused_in, proj)
            else:
                K.skinny_linear(x, self._fused_in, proj)
        # The mixers only share their input: the first runs on a side stream beside the others
        # (in a captured step the two become parallel branches of the graph).
        products = [None] * len(self.mixers)
        if side is not None:
            side.wait_stream(main)
            with torch.cuda.stream(side):
                m, (c0, c1) = self.mixers[0], self._fused_cols[0]
                products[0] = (m.pre_output(proj[:, c0:c1], ctx, cache), m.output_weight(), m.out_scale)
        for i, (m, (c0, c1)) in enumerate(zip(self.mixers, self._fused_cols)):
            if products[i] is None:
                products[i] = (m.pre_output(proj[:, c0:c1], ctx, cache), m.output_weight(), m.out_scale)
        if side is not None:
            main.wait_stream(side)
            if ahead:
                # The mixers' phase reads the caches and states at the memory's full rate; the products
                # that follow are latency-bound and leave it idle: the next layer's weights are
                # requested beside them (the side branch joins again at the next layer's mixers).
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    K.l2_prefetch(ahead)
        # h = (h + s0 * y0 W0^T) + s1 * y1 W1^T in one launch, then the feed-forward
        act = ws.alloc((T, self.ffn.intermediate_size), ctx.dtype) if self.ffn is not None else None
        if _CHAINED:
            phases = [("residual", products)]
            if self.ffn is not None:
                phases += [("swiglu", self.ffn_norm.weight, self.ffn_norm.eps, self.ffn.gate_up,
                            self.ffn.gate_multiplier, act),
                           ("residual", [(act, self.ffn.down, self.ffn.out_scale)])]
            K.skinny_chain(h, phases)
        else:
            def add_products(prods):
                if tensor_core and all(K.skinny_tc_supported("residual", px, pw) for px, pw, _ in prods):
                    K.skinny_tc_residual(h, prods)
                else:
                    K.skinny_residual(h, prods)

            add_products(products)
            if self.ffn is not None:
                if fused_norm:
                    K.skinny_swiglu_norm(h, self.ffn_norm.weight, self.ffn_norm.eps, self.ffn.gate_up,
                                         self.ffn.gate_multiplier, act)
                else:
                    K.add_rmsnorm(h, [], self.ffn_norm.weight, self.ffn_norm.eps, x)
                    if tensor_core and K.skinny_tc_supported("swiglu", x, self.ffn.gate_up, act):
                        K.skinny_tc_swiglu(x, self.ffn.gate_up, self.ffn.gate_multiplier, act)
                    else:
                        K.skinny_swiglu(x, self.ffn.gate_up, self.ffn.gate_multiplier, act)
                add_products([(act, self.ffn.down, self.ffn.out_scale)])
        ws.release(mark)

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        if self._few_tokens_path(ctx):
            self._forward_few_tokens(stream, ctx, cache)
            return
        ws = ctx.workspace
        mark = ws.mark()
        n = stream.normed(self.mixer_norm)
        if self._fused_in is not None:
            proj = ws.alloc((n.shape[0], self._fused_in.shape[0]), n.dtype)
            K.linear(n, self._fused_in, proj)
            # The mixers only share their input.  With several, the first runs on a side stream
            # beside the others (parallel branches of a captured step): a prompt portion's scan and
            # attention are each a chain of launches with few blocks, and together they fill the GPU.
            outs = [stream.take_branch() for _ in self.mixers]
            side = self._side_stream(proj.device) if len(self.mixers) > 1 and _PARALLEL_MIXERS else None
            main = torch.cuda.current_stream(proj.device)
            for i, (m, (c0, c1)) in enumerate(zip(self.mixers, self._fused_cols)):
                if i == 0 and side is not None:
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        m.forward_projected(proj[:, c0:c1], ctx, cache, outs[i])
                else:
                    m.forward_projected(proj[:, c0:c1], ctx, cache, outs[i])
            if side is not None:
                main.wait_stream(side)
            for m, out in zip(self.mixers, outs):
                stream.add(out, m.out_scale)
        else:
            for m in self.mixers:
                out = stream.take_branch()
                m.forward(n, ctx, cache, out)
                stream.add(out, m.out_scale)
        if self.ffn is not None:
            f = stream.normed(self.ffn_norm)
            out = stream.take_branch()
            self.ffn.forward(f, ctx, out)
            stream.add(out, self.ffn.out_scale)
        ws.release(mark)


register_arrangement("parallel_prenorm", ParallelPreNormBlock)
