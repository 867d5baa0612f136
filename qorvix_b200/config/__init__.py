from .model_config import ConfigError, LlamaConfig, ModelConfig, RopeScaling, read_config_json
from .registry import (architecture_of, load_config, lookup_architecture, register_architecture,
                       registered_architectures, unregister_architecture)
