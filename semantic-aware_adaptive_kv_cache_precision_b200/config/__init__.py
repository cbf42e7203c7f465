"""Typed configurations and the architecture registry."""

from .specs import (BandScaling, DecayAttentionSpec, OutputNormBlockSpec, ParallelMixerSpec,
                    SelectiveScanSpec, WindowSinkAttentionSpec)
from .specs import (AttentionSpec, BlockSpec, ClampedExpertSpec, ConfigError, DeltaRuleSpec,
                    DenseMLPSpec, DifferentialAttentionSpec, GatedMLPSpec, LatentAttentionSpec,
                    LayerCall, LogDistanceAttentionSpec, ModelSpec, NormSpec, RampScaling,
                    RotarySpec, RoutedExpertsSpec, SandwichBlockSpec, StreamBlockSpec)
from .registry import (architecture_name, config_from_dict, config_from_folder,
                       known_architectures, register_architecture)
from .qwen2 import Qwen2Config
from .tebonex import TebonexConfig
from .venanex import VenanexConfig
from .zodirax import ZodiraxConfig
from .gesuvik import GesuvikConfig

__all__ = ["AttentionSpec", "BlockSpec", "ConfigError", "DeltaRuleSpec", "DenseMLPSpec",
           "GatedMLPSpec", "LayerCall", "LogDistanceAttentionSpec", "ModelSpec", "NormSpec",
           "RotarySpec", "StreamBlockSpec", "ClampedExpertSpec", "DifferentialAttentionSpec",
           "LatentAttentionSpec", "RampScaling", "RoutedExpertsSpec", "SandwichBlockSpec",
           "BandScaling", "DecayAttentionSpec", "OutputNormBlockSpec", "ParallelMixerSpec",
           "SelectiveScanSpec", "WindowSinkAttentionSpec", "ZodiraxConfig", "GesuvikConfig",
           "Qwen2Config", "TebonexConfig", "VenanexConfig", "architecture_name", "config_from_dict",
           "config_from_folder", "known_architectures", "register_architecture"]
