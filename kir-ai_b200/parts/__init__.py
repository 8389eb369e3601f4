"""The parts a model is put together from (see ``base`` for the interfaces)."""
from .attention import GQAttention
from .base import (FeedForward, KVCacheNeed, Mixer, Norm, Part, PositionEncoding, Runtime, StateNeed, StreamCopy, WeightSpec)
from .block import Block
from .embedding import Embedding, OutputHead
from .experts import RoutedExperts
from .latent import LatentAttention
from .linear import Linear
from .matrix_memory import MatrixMemory
from .merge import StreamMerge
from .mlp import PlainMLP
from .mingru import MinGRU
from .norm import DynamicTanh, LayerNorm, RMSNorm
from .rope import RotaryEmbedding
from .shift import TokenShift
from .side_by_side import SideBySideMixer
from .state_space import StateSpaceMixer
from .swiglu import GatedMLP, SwiGLU

__all__ = ["GQAttention", "FeedForward", "KVCacheNeed", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
           "StateNeed", "StreamCopy", "WeightSpec", "RoutedExperts", "Block", "Embedding", "OutputHead", "Linear", "RMSNorm", "RotaryEmbedding", "SwiGLU",
           "GatedMLP", "LatentAttention", "LayerNorm", "MinGRU", "TokenShift", "DynamicTanh", "MatrixMemory", "SideBySideMixer",
           "StateSpaceMixer", "StreamMerge", "PlainMLP"]
