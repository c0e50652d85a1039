"""Typed configurations and the architecture registry."""

from .engine import EngineConfig
from .gigusun import ARCHITECTURE as GIGUSUN_ARCHITECTURE
from .gigusun import GigusunConfig
from .girelix import ARCHITECTURE as GIRELIX_ARCHITECTURE
from .girelix import GirelixConfig
from .kidarax import ARCHITECTURE as KIDARAX_ARCHITECTURE
from .kidarax import KidaraxConfig
from .lfm2 import ARCHITECTURE as LFM2_ARCHITECTURE
from .lfm2 import ConfigError, Lfm2Config
from .penopel import ARCHITECTURE as PENOPEL_ARCHITECTURE
from .penopel import PenopelConfig
from .registry import (
    architecture_of,
    architectures,
    config_from_dict,
    load_config,
    register_architecture,
)
from .specs import (
    AttentionSpec,
    DecayedLinearAttentionSpec,
    DynamicTanhSpec,
    GatedDeltaSpec,
    GatedLinearAttentionSpec,
    GatedMLPSpec,
    LatentAttentionSpec,
    LayerSpec,
    MLPSpec,
    ModelSpec,
    ParallelMixerSpec,
    PartSpec,
    PolyNormMLPSpec,
    RMSNormSpec,
    RopeSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
    ShortConvSpec,
    SwiGLUSpec,
)

register_architecture(LFM2_ARCHITECTURE, Lfm2Config, model_type="lfm2")
register_architecture(GIGUSUN_ARCHITECTURE, GigusunConfig)
register_architecture(GIRELIX_ARCHITECTURE, GirelixConfig)
register_architecture(PENOPEL_ARCHITECTURE, PenopelConfig)
register_architecture(KIDARAX_ARCHITECTURE, KidaraxConfig)

__all__ = [
    "AttentionSpec", "ConfigError", "DecayedLinearAttentionSpec", "DynamicTanhSpec", "GatedMLPSpec", "LatentAttentionSpec", "PenopelConfig", "GirelixConfig", "KidaraxConfig", "MLPSpec", "ParallelMixerSpec", "RoutedExpertsSpec", "EngineConfig", "GatedDeltaSpec", "GatedLinearAttentionSpec", "GigusunConfig", "LayerSpec",
    "Lfm2Config", "ModelSpec", "PartSpec", "PolyNormMLPSpec",
    "RMSNormSpec", "RopeSpec", "ScheduleEntry", "ShortConvSpec", "SwiGLUSpec", "architecture_of",
    "architectures", "config_from_dict", "load_config", "register_architecture",
]
