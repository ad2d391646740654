"""Model parts (mixers, feed-forwards, norms, position encodings, blocks), their registries, and
the model assembled from a spec."""

from .base import (BLOCKS, FEED_FORWARDS, INPUTS, MIXERS, NORMS, OUTPUTS, POSITION_ENCODINGS, Block, FeedForward,
                   InputPart, Mixer, Norm, OutputPart, Part, PositionEncoding, ResidualStream, StepContext, lookup,
                   register_block, register_feed_forward, register_input, register_mixer, register_norm,
                   register_output, register_position_encoding)
from . import norms, position, attention, feed_forward, blocks, ends  # noqa: F401  (registers the built-in kinds)
from .attention import Attention
from .blocks import PreNormResidual
from .ends import Embedding, NormHead
from .feed_forward import SwiGLU
from .model import Model, cache_specs, expected_weights, tile_requests
from .norms import RMSNorm
from .position import NoPosition, RopeNeox, rope_tables

__all__ = [
    "Attention", "BLOCKS", "Block", "Embedding", "FEED_FORWARDS", "FeedForward", "INPUTS", "InputPart", "MIXERS",
    "Mixer", "Model", "NORMS", "NoPosition", "Norm", "NormHead", "OUTPUTS", "OutputPart", "POSITION_ENCODINGS", "Part",
    "PositionEncoding", "PreNormResidual", "RMSNorm", "ResidualStream", "RopeNeox", "StepContext", "SwiGLU",
    "cache_specs", "expected_weights", "lookup", "register_block", "register_feed_forward", "register_input",
    "register_mixer", "register_norm", "register_output", "register_position_encoding",
    "rope_tables", "tile_requests",
]
