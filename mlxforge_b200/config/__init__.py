from .model_config import (ConfigError, LlamaConfig, ModelConfig, RopeScaling, read_config_json,
                           validate_rope_scaling, architecture_name)
from .registry import (Architecture, config_from_dir, config_from_json, get_architecture,
                       register_architecture, registered_architectures)
