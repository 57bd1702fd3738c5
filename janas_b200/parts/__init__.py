"""The parts a layer is put together from, and their registries."""
from .base import (DECODE, EXTEND, PREFILL, Block, FeedForward, LayerCache, Mixer, Norm, Part,
                   PositionEncoding, StepContext)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, block_class,
                       build_part, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position_encoding)
from . import norm, rope, attention, ffn, block  # register the built-in parts

__all__ = ["DECODE", "EXTEND", "PREFILL", "Block", "FeedForward", "LayerCache", "Mixer", "Norm",
           "Part", "PositionEncoding", "StepContext", "BLOCKS", "FEED_FORWARDS", "MIXERS",
           "NORMS", "POSITION_ENCODINGS", "block_class", "build_part", "register_block",
           "register_feed_forward", "register_mixer", "register_norm",
           "register_position_encoding"]
