"""Typed configuration and the architecture registry."""
from .specs import (AttentionSpec, BlockSpec, DecayAttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec,
                    LatentAttentionSpec, LayerRun, MlpSpec, MlstmSpec, ModelSpec, NormedEmbeddingSpec, NormSpec,
                    PairEmbeddingSpec, PositionSpec, RmsNormSpec, RotaryHalfSpec, RoutedExpertsSpec, StreamNormSpec,
                    WkvSpec)
from .registry import (architecture_names, config_class_for, config_from_dict, load_config,
                       register_architecture)
from .gptj import GptjConfig
from .lutelorn import LutelornConfig
from .fofinex import FofinexConfig

register_architecture(GptjConfig, GptjConfig.model_type)
register_architecture(LutelornConfig, LutelornConfig.model_type)
register_architecture(FofinexConfig, FofinexConfig.model_type)

__all__ = ["AttentionSpec", "BlockSpec", "DecayAttentionSpec", "EmbeddingSpec", "GatedMlpSpec", "HeadSpec",
           "LatentAttentionSpec", "LayerRun", "MlpSpec", "MlstmSpec", "ModelSpec", "NormedEmbeddingSpec", "NormSpec",
           "PairEmbeddingSpec", "PositionSpec", "RmsNormSpec", "RotaryHalfSpec", "RoutedExpertsSpec", "StreamNormSpec",
           "WkvSpec", "GptjConfig", "LutelornConfig", "FofinexConfig", "architecture_names",
           "config_class_for", "config_from_dict", "load_config", "register_architecture"]
