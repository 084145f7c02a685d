from .base import (ConfigError, ModelConfig, architecture_of, config_from_dict, describe_model,
                   known_architectures, load_config, register_architecture)
from .qwen3 import Qwen3Config
