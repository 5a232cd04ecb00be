from .attention import Attention
from .base import (Block, BuildOptions, FeedForward, HalfSum, KVSpec, Mixer, Norm, Part, PositionEncoding, StateSpec)
from .block import HiddenStream, ParallelBlock, PreNormBlock, SandwichBlock
from .embedding import PairTable, TokenEmbedding, VocabHead
from .experts import RoutedExperts
from .feedforward import SwiGLU
from .gated_recurrence import GatedDeltaRule, GatedLinearAttention
from .layer_norm import LayerNorm
from .latent_attention import LatentAttention
from .linear import Linear
from .linear_attention import DecayLinearAttention
from .maps_attention import MapsAttention
from .mlstm import MatrixMemory
from .norm import RMSNorm
from .side_by_side import SideBySide
from .position import RotaryEncoding, scaled_inv_freq
from .stream import PassOffset, TokenSide, TokenTable

__all__ = ["GatedDeltaRule", "GatedLinearAttention", "LayerNorm", "PairTable", "HalfSum", "SandwichBlock", "SideBySide", "Attention", "Block", "BuildOptions", "FeedForward", "KVSpec", "Mixer", "Norm", "Part", "PositionEncoding",
           "StateSpec", "HiddenStream", "PreNormBlock", "ParallelBlock", "RoutedExperts", "LatentAttention", "MatrixMemory", "TokenEmbedding", "VocabHead", "SwiGLU", "Linear",
           "RMSNorm", "RotaryEncoding", "scaled_inv_freq", "DecayLinearAttention", "MapsAttention", "PassOffset", "TokenSide",
           "TokenTable"]
