"""Typed configurations, part specifications and the architecture registry."""

from .errors import ConfigError, UnknownArchitectureError
from .lfm2 import Lfm2Config
from .plan import (
    AttentionSpec,
    BlockSpec,
    FeedForwardSpec,
    GatedDeltaSpec,
    GatedMLPSpec,
    LatentAttentionSpec,
    MixerSpec,
    ModelPlan,
    NormSpec,
    OutputNormBlockSpec,
    ParallelMixerSpec,
    PositionSpec,
    RMSNormSpec,
    RopeSpec,
    RoutedMLPSpec,
    SandwichBlockSpec,
    ScheduleEntry,
    ShortConvSpec,
)
from .tudulix import TudulixConfig
from .vuvulorn import VuvulornConfig
from .registry import architectures, config_from_dict, load_config, register_architecture

register_architecture("Lfm2ForCausalLM", Lfm2Config)
register_architecture("Vuvulorn", VuvulornConfig)
register_architecture("Tudulix", TudulixConfig)

__all__ = [
    "AttentionSpec",
    "BlockSpec",
    "ConfigError",
    "FeedForwardSpec",
    "GatedDeltaSpec",
    "GatedMLPSpec",
    "LatentAttentionSpec",
    "Lfm2Config",
    "MixerSpec",
    "ModelPlan",
    "NormSpec",
    "OutputNormBlockSpec",
    "ParallelMixerSpec",
    "PositionSpec",
    "RMSNormSpec",
    "RopeSpec",
    "RoutedMLPSpec",
    "SandwichBlockSpec",
    "ScheduleEntry",
    "ShortConvSpec",
    "TudulixConfig",
    "UnknownArchitectureError",
    "VuvulornConfig",
    "architectures",
    "config_from_dict",
    "load_config",
    "register_architecture",
]
