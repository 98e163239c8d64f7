"""Building blocks of a model: mixers, feed-forwards, norms, position encodings and the
arrangements that order them in a layer.  Importing the package registers the built-in
parts."""
from . import base
from .base import (FeedForward, LayerCache, LayerCall, LayerSpec, Mixer, ModelSpec, Norm, PagedView,
                   ParamSpec, Part, PartSpec, PositionEncoding, StateSpec, build_part,
                   register_arrangement, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding, register_stream_update, registered)
from . import streaming  # noqa: F401
from . import norm, rope, ffn, attention, mamba2, block  # noqa: F401  (registration)
from . import hyper, parallel, recurrent, window_attention  # noqa: F401  (registration)
from . import gated_attention, moe  # noqa: F401  (registration)
from . import latent_attention, stream_update  # noqa: F401  (registration)
from . import conv_attention  # noqa: F401  (registration)
from .block import ParallelPreNormBlock, ResidualStream, SharedNormParallelBlock, prenorm_layer, shared_norm_layer
