from .plan import ModelPlan, LayerSpec, OrderEntry, PartSpec, prenorm_layer
from .registry import register_architecture, known_architectures, detect, parse_config
from .lfm2 import Lfm2Config, ConfigError

register_architecture("Lfm2ForCausalLM", Lfm2Config.from_dict, model_types=("lfm2",))

__all__ = ["ModelPlan", "LayerSpec", "OrderEntry", "PartSpec", "prenorm_layer", "register_architecture", "known_architectures",
           "detect", "parse_config", "Lfm2Config", "ConfigError"]
