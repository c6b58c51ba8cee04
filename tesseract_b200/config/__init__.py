from .engine_config import EngineConfig
from .reading import ConfigError, NoArchitectureError, UnsupportedArchitectureError, read_config_json, require
from .registry import (Architecture, known_architectures, load_model_description, load_plugins, register_architecture,
                       resolve_architecture, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
