from .engine_config import EngineConfig
from .model_config import ConfigError, LlamaConfig, ModelConfig, RopeScaling
from .registry import (Architecture, config_from_dict, get_architecture, known_architectures, load_config,
                       model_spec, register_architecture)
