from .attention import Attention
from .base import KINDS, Part, make_part, register_part, registered
from .block import PreNormBlock, SandwichBlock
from .embedding import LMHead, TokenEmbedding
from .delta import ChannelDelta
from .diff_attention import DifferentialAttention
from .latent_attention import LatentAttention
from .mingru import MinGRU
from .token_mix import InputConv, TokenShift, TokenSide
from .moe import RoutedExperts
from .mlp import ClampedGLU, DenseMLP, GatedMLP, PolyNormMLP
from .norm import DynamicTanh, LayerNorm, PendingDelta, RMSNorm, UnitMix
from .parallel import ConvAttention, ParallelMixer, StateSpaceDual
from .sink_attention import SinkAttention
from .rope import NoPosition, Rope, RotaryPosition, frequency_factors, store_kv

__all__ = ["Attention", "KINDS", "Part", "make_part", "register_part", "registered", "PreNormBlock", "LMHead",
           "TokenEmbedding", "GatedMLP", "DenseMLP", "ClampedGLU", "RoutedExperts", "ChannelDelta", "SinkAttention", "DifferentialAttention", "LatentAttention", "MinGRU", "TokenShift", "TokenSide", "RMSNorm", "DynamicTanh", "LayerNorm", "PendingDelta", "UnitMix", "SandwichBlock", "InputConv", "PolyNormMLP", "ConvAttention", "ParallelMixer", "StateSpaceDual", "NoPosition", "Rope", "RotaryPosition", "frequency_factors", "store_kv"]
