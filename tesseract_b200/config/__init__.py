from .engine_config import EngineConfig
from .model_config import (ConfigError, LlamaConfig, NoArchitectureError, RopeScaling, UnsupportedArchitectureError,
                           read_config_json)
from .registry import (Architecture, known_architectures, load_model_description, register_architecture,
                       resolve_architecture, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
