"""The parts layers are put together from, their registries, and the decoder built of them."""
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward, KVView, Mixer, Norm, Part,
                   Position, StepContext, build_part, register_arrangement, register_feed_forward, register_mixer,
                   register_norm, register_position)
from .norm import LayerNorm, RMSNorm
from .position import NoPosition, RotaryHalf
from .stream_position import SinusoidAdd
from .input_conv import CausalConvAdd
from .attention import GQAAttention
from .attention_headmix import HeadMixAttention
from .mingru import MinGRU
from .feed_forward import DenseMLP, GatedMLP, SwiGLU
from .linear_attention import LinearAttention
from .attention_gated import GatedAttention
from .branch_sum import BranchSum
from .mixture import Mixture
from .attention_latent import LatentAttention
from .state_space import StateSpace
from .block import Layer, parallel, post_norm, pre_norm, sandwich
from .model import DecoderModel

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "FeedForward", "KVView", "Mixer", "Norm",
           "Part", "Position", "StepContext", "build_part", "register_arrangement", "register_feed_forward",
           "register_mixer", "register_norm", "register_position", "RMSNorm", "NoPosition", "RotaryHalf",
           "GQAAttention", "SwiGLU", "Layer", "pre_norm", "DecoderModel", "LayerNorm", "SinusoidAdd", "CausalConvAdd",
           "HeadMixAttention", "MinGRU", "DenseMLP", "parallel", "GatedMLP", "LinearAttention", "GatedAttention", "BranchSum", "Mixture",
           "LatentAttention", "StateSpace", "post_norm", "sandwich"]
