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
from typing import List, Optional, Tuple

import torch

from ..kernels import ops as K
from . import branches, streaming
from .base import (FeedForward, LayerCache, LayerSpec, Mixer, Norm, Part, PartSpec, StateSpec,
                   build_part, register_arrangement)
from .norm import fold_branches

Tensor = torch.Tensor


# The mixers of a layer on parallel streams in steps of many tokens too (PMM_PARALLEL_MIXERS=0: one
# after the other).
_PARALLEL_MIXERS = os.environ.get("PMM_PARALLEL_MIXERS", "1") == "1"


def prenorm_layer(prefix: str, mixer_norm: PartSpec, mixers, ffn_norm: Optional[PartSpec] = None,
                  ffn: Optional[PartSpec] = None) -> LayerSpec:
    """The LayerSpec of a ``parallel_prenorm`` layer: norm -> parallel mixers -> norm -> feed-forward."""
    return LayerSpec("parallel_prenorm", prefix, {"mixer_norm": mixer_norm, "mixers": tuple(mixers),
                                                  "ffn_norm": ffn_norm, "ffn": ffn})


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
        unknown = set(spec.parts) - {"mixer_norm", "mixers", "ffn_norm", "ffn"}
        if unknown or spec.part("mixer_norm") is None or not spec.part("mixers"):
            raise ValueError("parallel_prenorm takes the parts mixer_norm, mixers (at least one), ffn_norm and ffn"
                             + (f"; got also {sorted(unknown)}" if unknown else ""))
        self.mixer_norm: Norm = build_part("norm", spec.part("mixer_norm"), width=hidden_size)
        self.mixers: List[Mixer] = [build_part("mixer", m, hidden_size=hidden_size) for m in spec.part("mixers")]
        self.ffn_norm: Optional[Norm] = None
        self.ffn: Optional[FeedForward] = None
        if spec.part("ffn") is not None:
            if spec.part("ffn_norm") is None:
                raise ValueError("a feed-forward needs its norm")
            self.ffn_norm = build_part("norm", spec.part("ffn_norm"), width=hidden_size)
            self.ffn = build_part("feed_forward", spec.part("ffn"), hidden_size=hidden_size)
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
        weight-streaming products (norm in the prologue, the residual add in the epilogue) instead
        of library products with separate element-wise launches.  Needs mixers that share one
        input projection and expose their output projections; any norm and any feed-forward do
        (a feed-forward without a few-token path of its own runs its general `forward`)."""
        if not streaming.eligible(ctx, self.hidden_size) or self._fused_in is None:
            return False
        if any(m.output_weight() is None or m.output_bias() is not None for m in self.mixers):
            return False
        return len(self.mixers) <= 2

    @staticmethod
    def _side_stream(device: torch.device) -> "torch.cuda.Stream":
        return branches.branch_stream(device, "mixer")

    @staticmethod
    def _fetch_stream(device: torch.device) -> "torch.cuda.Stream":
        return branches.branch_stream(device, "fetch")

    def streamed_weights(self) -> List[Tensor]:
        """The matrices a step of few tokens reads once: what the layer before this one may
        ask the memory system to fetch ahead."""
        ws = [self._fused_in] + [m.output_weight() for m in self.mixers]
        if self.ffn is not None:
            ws += list(self.ffn.streamed_weights())
        return [w for w in ws if w is not None]

    def _forward_few_tokens(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        ws = ctx.workspace
        mark = ws.mark()
        h = stream.flush()
        T = h.shape[0]
        side = self._side_stream(h.device) if len(self.mixers) > 1 else None
        main = torch.cuda.current_stream(h.device)
        ahead = getattr(ctx, "fetch_ahead", None)  # the next layer's weights, set by the model
        proj = ws.alloc((T, self._fused_in.shape[0]), ctx.dtype)
        streaming.normed_linear(h, self.mixer_norm, self._fused_in, proj, ctx)
        # The mixers only share their input: the first runs on a side stream beside the others
        # (in a captured step the two become parallel branches of the graph).
        products = [None] * len(self.mixers)
        if side is not None:
            with branches.fork(main, side):
                m, (c0, c1) = self.mixers[0], self._fused_cols[0]
                products[0] = (m.pre_output(proj[:, c0:c1], ctx, cache), m.output_weight(), m.out_scale)
        for i, (m, (c0, c1)) in enumerate(zip(self.mixers, self._fused_cols)):
            if products[i] is None:
                products[i] = (m.pre_output(proj[:, c0:c1], ctx, cache), m.output_weight(), m.out_scale)
        if side is not None:
            main.wait_stream(side)
        if ahead:
            # The mixers' phase reads the caches and states at the memory's full rate; the products
            # that follow are latency-bound and leave it idle: the next layer's weights are requested
            # beside them.  On the mixers' side stream the next layer's first mixer queues behind the
            # fetch, which keeps the fetch out of that layer's mixer phase (measured on the 0.5B sizes,
            # ms a step with the fetch on the side stream / on a stream nothing waits for / without:
            # 8 tokens 1.03 / 1.04 / 1.07, 16 tokens 1.32 / 1.48 / 1.45); a step of one token has no
            # phase to protect and is faster when nothing waits (1.06 / 0.88 / 0.92).
            fetch = side if side is not None and T > 1 else self._fetch_stream(h.device)
            with branches.fork(main, fetch):
                K.l2_prefetch(ahead)
            ctx.unjoined_stream = fetch  # joined by the model when the step's last layer has run
        # h = (h + s0 * y0 W0^T) + s1 * y1 W1^T in one launch, then the feed-forward
        streaming.add_products(h, products, ctx)
        if self.ffn is not None and not self.ffn.forward_few_tokens(h, self.ffn_norm, ctx):
            f = stream.normed(self.ffn_norm)   # a feed-forward without a few-token path of its own
            out = stream.take_branch()
            self.ffn.forward(f, ctx, out)
            stream.add(out, self.ffn.out_scale)
        ws.release(mark)

    def accepts_length_bounds(self, dtype: torch.dtype, page_size: int) -> bool:
        """See Mixer.accepts_length_bounds: norms and feed-forwards go row by row, the mixers decide."""
        return all(m.accepts_length_bounds(dtype, page_size) for m in self.mixers)

    def joins_side_stream(self, ctx) -> bool:
        """Whether this layer may start while ``ctx.unjoined_stream`` still works (a weight fetch that
        an earlier layer of the same kind left running: nothing this layer does depends on it)."""
        return self._few_tokens_path(ctx)

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
                    with branches.fork(main, side):
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
