"""The parts a model is put together from: norms, position encodings, mixers,
feed-forwards and their arrangement in a block."""

from .base import Part, build_part, register_part
from .norm import LayerNorm, RMSNorm
from .rotary import NoPosition, RotaryHalf, RotaryInterleaved
from .attention import GQAAttention
from .mlp import DenseMLP, GatedMLP
from .block import PreNormBlock
from .delta_rule import DeltaRuleMixer
from .distance_attention import LogDistanceAttention
from .streams import StreamBlock, StreamUpdate
from .latent_attention import LatentAttention
from .differential_attention import DifferentialAttention
from .routed_experts import RoutedExperts
from .sandwich import NormedUpdate, SandwichBlock
from .window_sink_attention import WindowSinkAttention
from .decay_attention import DecayAttention
from .parallel_mixer import ParallelMixer
from .selective_scan import SelectiveScanMixer
from .output_norm import OutputNormBlock

__all__ = ["Part", "build_part", "register_part", "RMSNorm", "RotaryHalf", "RotaryInterleaved", "NoPosition",
           "GQAAttention", "GatedMLP", "DenseMLP", "PreNormBlock", "DeltaRuleMixer",
           "LogDistanceAttention", "StreamBlock", "StreamUpdate", "LayerNorm", "LatentAttention",
           "DifferentialAttention", "RoutedExperts", "SandwichBlock", "NormedUpdate",
           "WindowSinkAttention", "DecayAttention", "ParallelMixer", "SelectiveScanMixer",
           "OutputNormBlock"]
