"""A model assembled from a ModelSpec: embedding, layers (arrangements of parts), the
order in which the layers run, final norm and output head.

The forward pass is the same for every architecture:
  h = multiplier * E[tokens]                       (float32 residual stream)
  for (layer, cache_of) in order: layers[layer](h, cache of cache_of)
  logits = (norm(h)[wanted rows] @ W_head^T) * head_multiplier       (float32)
(reference src/runtime/runner/falconh1_runner.cpp:129-228, which keeps the last row only).
"""
from __future__ import annotations

import os

from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops as K
from ..parts.base import LayerCache, ModelSpec, ParamSpec, Part, StateSpec, build_part, _REGISTRIES
from ..parts.block import ResidualStream
from .context import StepContext

# The output head of steps with few wanted rows through the weight-streaming product (PMM_SKINNY_HEAD=0:
# the library product).
_SKINNY_HEAD = os.environ.get("PMM_SKINNY_HEAD", "1") == "1"
_FETCH_FROM_TOKENS, _FETCH_TO_TOKENS = 1, 16

Tensor = torch.Tensor


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.layers = []
        self._fetch_ahead = os.environ.get("PMM_FETCH_AHEAD", "1") == "1"
        self._fetch_lists: Dict[int, tuple] = {}
        for ls in spec.layers:
            factory = _REGISTRIES["arrangement"].get(ls.arrangement)
            if factory is None:
                raise KeyError(f"unknown arrangement '{ls.arrangement}'")
            self.layers.append(factory(ls, hidden_size=spec.hidden_size))
        for call in spec.order:
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"execution order names a layer that does not exist: {call}")
        self.final_norm = build_part("norm", spec.final_norm, width=spec.hidden_size)
        self.embedding: Optional[Tensor] = None
        self.head: Optional[Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._branch_buffers = max(l.branch_buffers_needed() for l in self.layers) if self.layers else 1

    # ------------------------------------------------------------------ tensors
    def named_parts(self) -> List[Tuple[str, Part]]:
        """(name prefix, part) for every part that owns tensors."""
        out: List[Tuple[str, Part]] = []
        for layer in self.layers:
            for part in layer.parts():
                out.append((f"{layer.prefix}{part.name}.", part))
        out.append((f"{self.spec.final_norm.name}.", self.final_norm))
        return out

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs: Dict[str, ParamSpec] = {
            self.spec.embedding_name: ParamSpec(self.spec.embedding_name,
                                                (self.vocab_size, self.hidden_size)),
        }
        if self.spec.head_name is not None:
            specs[self.spec.head_name] = ParamSpec(self.spec.head_name, (self.vocab_size, self.hidden_size))
        for prefix, part in self.named_parts():
            for ps in part.param_specs():
                specs[prefix + ps.name] = ps
        return specs

    def ignored_names(self) -> List[str]:
        names: List[str] = []
        for prefix, part in self.named_parts():
            names += [prefix + n for n in getattr(part, "ignored_names", lambda: [])()]
        return names

    def bind(self, tensors: Dict[str, Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """``tensors``: full name -> tensor on ``device`` in the policy type of its spec."""
        self.dtype, self.device = dtype, torch.device(device)
        self.embedding = tensors[self.spec.embedding_name]
        self.head = self.embedding if self.spec.head_name is None else tensors[self.spec.head_name]
        for prefix, part in self.named_parts():
            part.bind({ps.name: tensors[prefix + ps.name] for ps in part.param_specs()})
        for layer in self.layers:
            layer.finalize(dtype, self.device)
        self.final_norm.finalize(dtype, self.device)

    # ------------------------------------------------------------------ state
    def state_specs(self) -> Dict[int, List[Tuple[str, StateSpec]]]:
        """Cache id -> (qualified name, spec) of every state kept under it.  A cache id is what
        the execution order's ``cache_of`` names: the states that the layers run with that id
        declare, each name once (a layer that only reads another's state declares none)."""
        out: Dict[int, List[Tuple[str, StateSpec]]] = {}
        for call in self.spec.order:
            have = out.setdefault(call.cache_of, [])
            for name, spec in self.layers[call.layer].state_specs():
                known = dict(have)
                if name in known:
                    if known[name] != spec:
                        raise ValueError(f"cache {call.cache_of}: state '{name}' declared with two layouts")
                    continue
                have.append((name, spec))
        return out

    # ------------------------------------------------------------------ the step
    def forward(self, ctx: StepContext, caches: Dict[int, LayerCache]) -> Tensor:
        """Runs the step's tokens through the layers; returns logits [n_rows, V] float32 (taken
        from the step's workspace: valid until the workspace is reset by the next step)."""
        ws = ctx.workspace
        T, D = ctx.n_tokens, self.hidden_size
        h = ws.alloc((T, D), torch.float32)
        K.embed(h, self.embedding, ctx.tokens, self.spec.embedding_multiplier)
        stream = ResidualStream(h, ctx, self._branch_buffers)
        order = self.spec.order
        # Fetching the next layer's weights beside a layer's products pays where the mixers' phase is
        # long enough to cover it and the products still wait for their weights: measured on the 0.5B
        # sizes it takes 4 to 9 % off steps of up to 16 tokens and adds 1 % beyond 24.
        fetch = self._fetch_ahead and _FETCH_FROM_TOKENS <= T <= _FETCH_TO_TOKENS
        for i, call in enumerate(order):
            # a layer that streams its weights once may fetch the next layer's ahead of time
            nxt = self.layers[order[i + 1].layer] if i + 1 < len(order) else None
            ctx.fetch_ahead = self._weights_to_fetch(nxt, h.device) if fetch else None
            layer = self.layers[call.layer]
            if ctx.unjoined_stream is not None and not getattr(layer, "joins_side_stream", lambda c: False)(ctx):
                self._join(ctx, h.device)
            layer.forward(stream, ctx, caches[call.cache_of])
        ctx.fetch_ahead = None
        self._join(ctx, h.device)
        if ctx.n_rows == 0:
            stream.flush()
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=h.device)
        normed = stream.normed(self.final_norm, rows=ctx.logit_rows)
        return self._head(normed, ctx)

    def accepts_length_bounds(self, page_size: int) -> bool:
        """Whether every layer stays right when a step's lengths are given as bounds (see
        Mixer.accepts_length_bounds); an arrangement that does not say so does not."""
        return self.dtype is not None and all(
            getattr(layer, "accepts_length_bounds", lambda d, p: False)(self.dtype, page_size) for layer in self.layers)

    @staticmethod
    def _join(ctx: StepContext, device) -> None:
        """Wait for what a layer left running on a side stream (so that a recorded step ends joined)."""
        if ctx.unjoined_stream is not None:
            torch.cuda.current_stream(device).wait_stream(ctx.unjoined_stream)
            ctx.unjoined_stream = None

    def _weights_to_fetch(self, layer, device) -> Optional[List[Tensor]]:
        """The matrices of ``layer`` to request into L2 while the layer before it runs, or None.
        Only a layer whose matrices take at most a third of the L2 is fetched ahead: measured
        +4% tokens/s at 26 MB a layer, nothing at 50 MB, and -16% at 365 MB (the lines are
        evicted before they are used, and read twice)."""
        if layer is None or not hasattr(layer, "streamed_weights"):
            return None
        cached = self._fetch_lists.get(id(layer))
        if cached is None:
            ws = layer.streamed_weights()
            l2 = torch.cuda.get_device_properties(device).L2_cache_size if device.type == "cuda" else 0
            size = sum(w.numel() * w.element_size() for w in ws)
            cached = (ws if 0 < size <= l2 // 3 else None,)
            self._fetch_lists[id(layer)] = cached
        return cached[0]

    def _head_row_group(self, n_rows: int) -> int:
        """Rows per launch of the weight-streaming head product, or 0 for the library product.
        Measured (table read once, 8..64 rows): with a vocabulary that is a multiple of 8 the
        library reads the table at 3 TB/s and wins from 17 rows on (23 vs 32 us at 32,784 x 1,024);
        with any other vocabulary it falls to a slow kernel (163 vs 62 us at 65,537 x 1,280 and 32
        rows; 780 vs 176 us at 130,049 x 3,072), so there the streaming product is used even when
        the rows need up to four passes over the table."""
        D = self.hidden_size
        if D % 8:
            return 0
        group = next((m for m in (64, 32, 16, 8) if K.skinny_fits(m, D)), 0)
        if group == 0:
            return 0
        if n_rows <= min(group, K.SKINNY_NORM_MAX_TOKENS):
            return n_rows
        passes = -(-n_rows // group)
        return group if self.vocab_size % 8 and passes <= 4 else 0

    def _head(self, normed: Tensor, ctx: StepContext) -> Tensor:
        n_rows, V = normed.shape[0], self.vocab_size
        ws = ctx.workspace
        logits = ws.alloc((n_rows, V), torch.float32)
        mult = self.spec.head_multiplier
        if normed.dtype == torch.float32:
            K.linear(normed, self.head, logits)
            if mult != 1.0:
                K.scale_f32_(logits, mult)
        elif _SKINNY_HEAD and self._head_row_group(n_rows) > 0:
            # the table is read at memory speed by this repository's weight-streaming product
            # (float32 out, multiplier in the epilogue), once per group of rows that fits its shared memory
            group = self._head_row_group(n_rows)
            for r0 in range(0, n_rows, group):
                K.skinny_linear_f32(normed[r0:r0 + group], self.head, logits[r0:r0 + group], mult)
        else:
            low = None if K.mm_has_f32_out() else ws.alloc((n_rows, V), normed.dtype)
            K.linear_f32_out(normed, self.head, logits, low, mult)
        return logits
