"""Parts a layer is put together from: mixers, feed-forwards, norms, position encodings,
and their arrangement in a block.  Importing this package registers the built-in kinds."""
from .base import (
    BuildEnv, DeferredNorm, FeedForward, Mixer, Norm, Part, PositionEncoding, ResidualSink, build_block,
    build_feed_forward,
    build_mixer, build_norm, build_position, register_arrangement, register_feed_forward,
    register_mixer, register_norm, register_position, registered,
)
from .linear import Linear
from .norm import RMSNorm
from .position import NoPosition, RotaryNeox
from .attention import Attention
from .mlp import GatedMLP
from .block import PreNormBlock

__all__ = [
    "BuildEnv", "DeferredNorm", "ResidualSink", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "build_block",
    "build_feed_forward", "build_mixer", "build_norm", "build_position", "register_arrangement",
    "register_feed_forward", "register_mixer", "register_norm", "register_position", "registered",
    "Linear", "RMSNorm", "NoPosition", "RotaryNeox", "Attention", "GatedMLP", "PreNormBlock",
]
