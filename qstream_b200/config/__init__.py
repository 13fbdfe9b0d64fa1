"""Typed configuration and the architecture registry."""
from .specs import (AttentionSpec, BlockSpec, DecayAttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LayerRun,
                    MlpSpec, ModelSpec, NormSpec, PairEmbeddingSpec, PositionSpec, RmsNormSpec, WkvSpec)
from .registry import (architecture_names, config_class_for, config_from_dict, load_config,
                       register_architecture)
from .gptj import GptjConfig
from .lutelorn import LutelornConfig

register_architecture(GptjConfig, GptjConfig.model_type)
register_architecture(LutelornConfig, LutelornConfig.model_type)

__all__ = ["AttentionSpec", "BlockSpec", "DecayAttentionSpec", "EmbeddingSpec", "GatedMlpSpec", "HeadSpec", "LayerRun",
           "MlpSpec", "ModelSpec", "NormSpec", "PairEmbeddingSpec", "PositionSpec", "RmsNormSpec", "WkvSpec",
           "GptjConfig", "LutelornConfig", "architecture_names",
           "config_class_for", "config_from_dict", "load_config", "register_architecture"]
