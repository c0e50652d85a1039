"""Mixers, feed-forwards, norms, position encodings, and the block that arranges them."""

from .base import (
    FeedForward,
    Mixer,
    Normed,
    PagedKVSpec,
    PagedLatentSpec,
    PagedSpec,
    Param,
    Part,
    Runtime,
    StateSpec,
    build_part,
    project,
    project_swiglu,
    register_ffn,
    register_mixer,
    register_norm,
    register_position,
)
from .attention import Attention
from .block import ARRANGEMENTS, Block
from .gated_mlp import GatedMLP
from .latent import LatentAttention
from .mlp import MLP
from .moe import RoutedExperts
from .norm import DynamicTanh, RMSNorm
from .parallel import ParallelMixer
from .polynorm import PolyNormMLP
from .recurrent import DecayedLinearAttention, GatedDelta, GatedLinearAttention
from .rope import Rope
from .shortconv import ShortConv
from .swiglu import SwiGLU

__all__ = [
    "ARRANGEMENTS", "MLP", "Attention", "Block", "DynamicTanh", "GatedMLP", "LatentAttention", "PagedLatentSpec", "DecayedLinearAttention", "ParallelMixer", "RoutedExperts", "FeedForward", "GatedDelta", "GatedLinearAttention", "Mixer", "PolyNormMLP", "Normed", "PagedKVSpec", "PagedSpec", "Param", "Part", "RMSNorm",
    "Rope", "Runtime", "ShortConv", "StateSpec", "SwiGLU", "build_part", "project", "project_swiglu", "register_ffn", "register_mixer",
    "register_norm", "register_position",
]
