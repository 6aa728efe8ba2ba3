from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (architecture_name, load_config, parse_config, register_architecture,
                       registered_architectures)
from .qwen2 import Qwen2Config
from .tulipel import TulipelConfig
from .letanex import LetanexConfig
from .rarutar import RarutarConfig
from .vuripel import VuripelConfig

register_architecture(Qwen2Config.architecture, Qwen2Config, model_types=(Qwen2Config.model_type,))
register_architecture(TulipelConfig.architecture, TulipelConfig)
register_architecture(LetanexConfig.architecture, LetanexConfig)
register_architecture(RarutarConfig.architecture, RarutarConfig)
register_architecture(VuripelConfig.architecture, VuripelConfig)

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config", "TulipelConfig", "LetanexConfig", "RarutarConfig", "VuripelConfig",
           "architecture_name", "load_config", "parse_config", "register_architecture",
           "registered_architectures"]
