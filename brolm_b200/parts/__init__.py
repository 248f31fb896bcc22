from .attention import Attention
from .base import ParamSpec, Part, PartSpec, part_class, register_part, registered_parts
from .block import Block, BlockSpec
from .feedforward import GatedFeedForward
from .layout import EmbeddingSpec, HeadSpec, LayerCall, ModelLayout
from .linear import linear
from .norm import RMSNorm, add_then_norm
from .position import RotaryEmbedding

__all__ = ["Attention", "ParamSpec", "Part", "PartSpec", "part_class", "register_part", "registered_parts", "Block",
           "BlockSpec", "GatedFeedForward", "EmbeddingSpec", "HeadSpec", "LayerCall", "ModelLayout", "linear",
           "RMSNorm", "add_then_norm", "RotaryEmbedding"]
