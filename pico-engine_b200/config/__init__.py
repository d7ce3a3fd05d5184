"""Typed configurations, part descriptions and the architecture registry."""
from .specs import (ConfigError, PartSpec, RMSNormSpec, LayerNormSpec, RotaryHalfSpec, NoPositionSpec, SinusoidAddSpec,
                    CausalConvAddSpec, GQAAttentionSpec, HeadMixAttentionSpec, MinGRUSpec, SwiGLUSpec, DenseMLPSpec,
                    LayerSpec, ScheduleEntry, ModelPlan, RotaryPairsSpec, GatedAttentionSpec, LinearAttentionSpec, BranchSumSpec,
                    GatedMLPSpec, MixtureSpec, LatentAttentionSpec, StateSpaceSpec, BigramTableSpec, RotaryHalvesSpec)
from .registry import (Architecture, register_architecture, known_architectures, architecture,
                       architecture_name_of, config_from_dict, read_config)
from .qwen2 import Qwen2Config
from .mebalorn import MebalornConfig
from .kevelorn import KevelornConfig
from .pupidra import PupidraConfig
from .tenusun import TenusunConfig

__all__ = ["ConfigError", "PartSpec", "RMSNormSpec", "LayerNormSpec", "RotaryHalfSpec", "NoPositionSpec",
           "SinusoidAddSpec", "CausalConvAddSpec", "GQAAttentionSpec", "HeadMixAttentionSpec", "MinGRUSpec",
           "SwiGLUSpec", "DenseMLPSpec", "MebalornConfig", "LayerSpec", "ScheduleEntry", "ModelPlan", "Architecture", "register_architecture",
           "known_architectures", "architecture", "architecture_name_of", "config_from_dict", "read_config",
           "Qwen2Config", "KevelornConfig", "RotaryPairsSpec", "GatedAttentionSpec", "LinearAttentionSpec", "BranchSumSpec",
           "GatedMLPSpec", "MixtureSpec", "LatentAttentionSpec", "StateSpaceSpec", "BigramTableSpec", "PupidraConfig", "RotaryHalvesSpec", "TenusunConfig"]
