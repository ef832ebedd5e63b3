"""Configuration: typed reading of config.json and the architecture registry."""
from .base import ConfigError, KeyReader, read_config_json
from .spec import (AdapterSpec, AttentionSpec, FeedForwardSpec, GatedMLPSpec, LayerSpec, MixerSpec,
                   ModelSpec, NormSpec, PositionSpec, RunStep)
from .registry import (Architecture, find_architecture, load_config, register_architecture,
                       registered_architectures, unregister_architecture)
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE, MODEL_TYPE as QWEN3_MODEL_TYPE, Qwen3Config

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config.from_dict, Qwen3Config.model_spec,
                      model_type=QWEN3_MODEL_TYPE, replace=True)

__all__ = [
    "ConfigError", "KeyReader", "read_config_json",
    "AdapterSpec", "AttentionSpec", "FeedForwardSpec", "GatedMLPSpec", "LayerSpec", "MixerSpec", "ModelSpec",
    "NormSpec", "PositionSpec", "RunStep",
    "Architecture", "find_architecture", "load_config", "register_architecture",
    "registered_architectures", "unregister_architecture", "Qwen3Config",
]
