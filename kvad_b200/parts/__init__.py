"""Parts: position encodings, norms, mixers, feed-forwards, block arrangements, ends."""
from .base import (FAMILIES, Block, FeedForward, Mixer, Norm, Part, PartSpec, PositionEncoding,
                   build_part, part_kinds, register_part, unregister_part)
from .linear import Linear
from . import norms, positions, attention, feedforward, block, ends  # noqa: F401  (register the built-in kinds)
from .norms import LayerNorm
from .positions import LearnedAbsolute, NoPositions
from .attention import CausalSelfAttention
from .feedforward import DenseMLP
from .block import PreNormBlock
from .ends import LMHead, TokenEmbedding

__all__ = [
    "FAMILIES", "Block", "FeedForward", "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding",
    "build_part", "part_kinds", "register_part", "unregister_part", "Linear", "LayerNorm",
    "LearnedAbsolute", "NoPositions", "CausalSelfAttention", "DenseMLP", "PreNormBlock", "LMHead",
    "TokenEmbedding",
]
