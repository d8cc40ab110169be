"""Building blocks of a model: mixers, feed-forwards, norms, position encodings and the
arrangements that order them in a layer.  Importing the package registers the built-in
parts."""
from . import base
from .base import (FeedForward, LayerCache, LayerCall, LayerSpec, Mixer, ModelSpec, Norm, PagedView,
                   ParamSpec, Part, PartSpec, PositionEncoding, StateSpec, build_part,
                   register_arrangement, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding, registered)
from . import streaming  # noqa: F401
from . import norm, rope, ffn, attention, mamba2, block  # noqa: F401  (registration)
from .block import ParallelPreNormBlock, ResidualStream, prenorm_layer
