"""Interfaces of the building blocks and the registries they are chosen from.

A model is put together from *parts*: mixers (attention, state-space, ...),
feed-forwards, norms, position encodings, and *arrangements* that order them inside a
layer.  A part knows its own sizes and constants (all constructor parameters), the
tensors it needs (``param_specs``) and, for mixers, the per-request state it keeps
(``state_specs``).  It never knows which model it is in.  Architectures describe their
layers as data (``PartSpec`` / ``LayerSpec`` / ``ModelSpec``) and the registries below
turn the names into parts, so a new part is one ``register_*`` call away.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

Tensor = torch.Tensor


# ----------------------------------------------------------------------------- tensors a part needs
@dataclass(frozen=True)
class ParamSpec:
    """One tensor of a part.  ``name`` is relative to the part's prefix.

    kind: "matrix"  -> kept in the compute type (bfloat16 or float32);
          "vector"  -> always float32 on the device (norm weights, biases, per-head scalars);
          "table"   -> integer table, int32.
    init: how the random-weights mode fills it: ("normal", std) | ("ones",) | ("zeros",) |
          ("log_uniform", lo, hi) [log of U(lo,hi)] | ("inv_softplus_log_uniform", lo, hi).
    alt_shapes: other stored shapes with the same element count that are accepted and
          viewed as ``shape`` (e.g. a conv weight stored [C, 1, K]).
    stored_shape: shape written by the random-weights mode (defaults to ``shape``).
    """
    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: Tuple[Any, ...] = ("normal", 0.02)
    alt_shapes: Tuple[Tuple[int, ...], ...] = ()
    stored_shape: Optional[Tuple[int, ...]] = None


# ----------------------------------------------------------------------------- state a mixer keeps
@dataclass(frozen=True)
class StateSpec:
    """Per-request state of one mixer in one layer.

    kind "paged": ``planes`` rows of ``width`` elements per token (keys and values: 2
    planes), kept in pages through a block table; ``window`` > 0 means only the last
    ``window`` tokens are ever read, so older pages can be given back.
    kind "fixed": one tensor of ``shape`` per request, kept in a slot; zero for a new
    request.  dtype "compute" follows the engine's storage type, "float32" stays 32-bit.
    """
    name: str
    kind: str
    planes: int = 0
    width: int = 0
    window: int = 0
    shape: Tuple[int, ...] = ()
    dtype: str = "compute"

    @staticmethod
    def paged(name: str, planes: int, width: int, window: int = 0) -> "StateSpec":
        return StateSpec(name=name, kind="paged", planes=planes, width=width, window=window)

    @staticmethod
    def fixed(name: str, shape: Sequence[int], dtype: str = "float32") -> "StateSpec":
        return StateSpec(name=name, kind="fixed", shape=tuple(int(s) for s in shape), dtype=dtype)


@dataclass
class PagedView:
    """A layer's pages [num_pages, planes, page_size, width] with the step's block table
    [n_seq, max_blocks] (device int32; entries of pages given back are -1)."""
    pool: Tensor
    block_table: Tensor
    page_size: int
    window: int


class LayerCache:
    """What one layer's mixers see of the cache during a step: name -> PagedView or the
    slot tensor [num_slots, *shape] (indexed with the step's slot ids)."""

    def __init__(self, paged: Dict[str, PagedView], fixed: Dict[str, Tensor]):
        self._paged = paged
        self._fixed = fixed

    def paged(self, name: str) -> PagedView:
        return self._paged[name]

    def fixed(self, name: str) -> Tensor:
        return self._fixed[name]


# ----------------------------------------------------------------------------- parts
class Part:
    """Base of every part.  ``name`` is the part's component of tensor names."""

    name: str = ""

    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, params: Dict[str, Tensor]) -> None:
        """Receives the tensors of ``param_specs`` (by relative name) on the device."""
        self.params = params

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        """Called once after ``bind``: precompute tables, fuse, validate sizes against kernels."""


class Norm(Part):
    """forward(h, pending, out, rows, ctx): fold the pending branches [(tensor, scale), ...]
    into the float32 stream h (when rows is None) and write the normalised rows to out."""

    def forward(self, h: Tensor, pending, out: Tensor, rows: Optional[Tensor], ctx) -> None:
        raise NotImplementedError

    def rms_prologue(self) -> Optional[Tuple[Tensor, float]]:
        """(weight [D] float32, eps) if this norm is y = x / sqrt(mean(x^2) + eps) * weight, which
        the weight-streaming products of few-token steps can apply in their prologue; None for any
        other norm (it is then launched on its own through `forward`)."""
        return None


class PositionEncoding(Part):
    """Applied by a mixer to its queries and keys at absolute positions."""


class Mixer(Part):
    """Token mixer.  ``out_scale`` multiplies its output when it joins the residual stream.

    forward(x, ctx, cache, out): x [T, D] normalised activations of all tokens of the step,
    cache the LayerCache of the layer whose state it uses, out [T, D] to be written.

    A mixer whose first operation is a plain projection of x may expose it
    (``input_rows`` > 0, ``input_weight``) so that an arrangement can run the projections
    of parallel mixers as one matrix product and call ``forward_projected`` with the
    mixer's column slice instead.
    """
    out_scale: float = 1.0

    def state_specs(self) -> List[StateSpec]:
        return []

    def input_rows(self) -> int:
        return 0

    def input_weight(self) -> Tensor:
        raise NotImplementedError

    def adopt_input_weight(self, view: Tensor) -> None:
        raise NotImplementedError

    def forward(self, x: Tensor, ctx, cache: LayerCache, out: Tensor) -> None:
        raise NotImplementedError

    def forward_projected(self, proj: Tensor, ctx, cache: LayerCache, out: Tensor) -> None:
        raise NotImplementedError

    # A mixer whose last operation is a plain projection back to the stream may also expose
    # that: ``pre_output`` returns the activation [T, inner] that ``output_weight`` [D, inner]
    # is applied to (``output_bias`` [D] or None), so that an arrangement can run the output
    # projections of its mixers as one product that accumulates into the residual stream.
    def pre_output(self, proj: Tensor, ctx, cache: LayerCache) -> Tensor:
        raise NotImplementedError

    def output_weight(self) -> Optional[Tensor]:
        return None

    def output_bias(self) -> Optional[Tensor]:
        return None

    def accepts_length_bounds(self, dtype: torch.dtype, page_size: int) -> bool:
        """Whether this mixer's launches stay right when ``ctx.new_lens`` is not the true list of
        tokens per sequence but a list of the same length and sum chosen so that every count
        derived from it (chunks or tiles of any size, sequences of one token or of several) is an
        upper bound of the true one, the true lengths being in ``ctx.cu_seqlens`` on the device
        (some of them may be zero: sequences that bring no token must be left alone): kernels sized
        by such counts must let their surplus blocks leave.  Steps of recurring
        rounded shapes are then recorded once and replayed whatever the cut (see ModelRunner)."""
        return False


class FeedForward(Part):
    """forward(x, ctx, out): x [T, D] normalised activations, out [T, D]."""
    out_scale: float = 1.0

    def forward(self, x: Tensor, ctx, out: Tensor) -> None:
        raise NotImplementedError

    # Optional path for steps of few tokens in bfloat16, where every product is a read of its
    # weights.  An arrangement that takes that path for its mixers asks the feed-forward to do the
    # same: ``forward_few_tokens(h, norm, ctx)`` adds out_scale * ffn(norm(h)) into the float32
    # stream h [T, D] in place, with the operations of parts/streaming.py (norm in the prologue of
    # the first product, the residual add in the epilogue of the last), and returns True; the
    # default declines and the arrangement runs `forward` on the general path.
    def forward_few_tokens(self, h: Tensor, norm: "Norm", ctx) -> bool:
        return False

    def streamed_weights(self) -> List[Tensor]:
        """The matrices a few-token step reads once (what the layer before may fetch ahead)."""
        return []


# ----------------------------------------------------------------------------- specs (data)
@dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, its weight-name component and its constructor parameters."""
    kind: str
    name: str = ""
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer as data: the arrangement that orders its parts, the prefix of its tensor names,
    and the part specs under the names the arrangement defines (a PartSpec, a tuple of them, or
    None).  ``parallel_prenorm`` reads "mixer_norm", "mixers", "ffn_norm" and "ffn"
    (`parts.block.prenorm_layer` builds such a spec); another arrangement (post-norms, sandwich
    norms, two feed-forwards) names its own."""
    arrangement: str
    prefix: str
    parts: Mapping[str, Any] = field(default_factory=dict)

    def part(self, name: str, default: Any = None) -> Any:
        return self.parts.get(name, default)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the execution order: run ``layer`` on the cache of ``cache_of``
    (its own unless it reads another layer's)."""
    layer: int
    cache_of: int


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding_name: str
    embedding_multiplier: float
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: PartSpec
    head_name: Optional[str]  # None: tied to the embedding table
    head_multiplier: float
    eos_token_id: int = -1
    bos_token_id: int = 0


# ----------------------------------------------------------------------------- registries
_REGISTRIES: Dict[str, Dict[str, Callable[..., Part]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "arrangement": {},
}


def _register(family: str, kind: str, factory: Callable[..., Any]) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and reg[kind] is not factory:
        raise ValueError(f"{family} '{kind}' is already registered")
    reg[kind] = factory


def register_mixer(kind: str, factory: Callable[..., Mixer]) -> None:
    _register("mixer", kind, factory)


def register_feed_forward(kind: str, factory: Callable[..., FeedForward]) -> None:
    _register("feed_forward", kind, factory)


def register_norm(kind: str, factory: Callable[..., Norm]) -> None:
    _register("norm", kind, factory)


def register_position_encoding(kind: str, factory: Callable[..., PositionEncoding]) -> None:
    _register("position_encoding", kind, factory)


def register_arrangement(kind: str, factory: Callable[..., Any]) -> None:
    _register("arrangement", kind, factory)


def build_part(family: str, spec: PartSpec, **extra: Any) -> Any:
    """Instantiate ``spec`` from the registry of ``family``; the factory receives the
    spec's params plus ``name`` and whatever the caller adds (e.g. hidden_size)."""
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise KeyError(f"unknown {family} '{spec.kind}' (registered: {sorted(reg)})")
    part = reg[spec.kind](**extra, **spec.params)
    part.name = spec.name
    return part


def registered(family: str) -> List[str]:
    return sorted(_REGISTRIES[family])
