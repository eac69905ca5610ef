"""Typed configuration: part records (``specs``) and the architecture registry."""
from .specs import (AttentionSpec, DenseFFSpec, EmbeddingSpec, GLASpec, HeadSpec, HyperConnectionSpec,
                    LatentAttentionSpec, LayerNormSpec, LayerSpec, ModelSpec, NoPositionSpec, RMSNormSpec, RopePairsSpec,
                    RopeSpec, ScheduleEntry, StreamLayerSpec, SwiGLUSpec)
from .registry import (ConfigError, UnsupportedArchitecture, architecture_of, config_from_dict,
                       load_config, register_architecture, registered_architectures)

__all__ = [
    "AttentionSpec", "DenseFFSpec", "EmbeddingSpec", "GLASpec", "HeadSpec", "HyperConnectionSpec", "LatentAttentionSpec",
    "LayerNormSpec", "LayerSpec", "ModelSpec", "NoPositionSpec", "RMSNormSpec", "RopePairsSpec", "RopeSpec",
    "ScheduleEntry", "StreamLayerSpec", "SwiGLUSpec", "ConfigError", "UnsupportedArchitecture", "architecture_of",
    "config_from_dict", "load_config", "register_architecture", "registered_architectures",
]
