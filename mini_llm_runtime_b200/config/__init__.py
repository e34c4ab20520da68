from .qwen2 import Qwen2Config, qwen2_model_spec
from .registry import (Architecture, architecture_of, config_from_dict, known_architectures,
                       load_config, register_architecture, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

__all__ = [
    "Architecture", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config", "RunStep",
    "architecture_of", "config_from_dict", "known_architectures", "load_config",
    "qwen2_model_spec", "register_architecture", "unregister_architecture",
]
