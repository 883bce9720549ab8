from .base import ConfigError, ModelConfig, key, load_stop_ids, read_config_json  # noqa: F401
from .registry import (Architecture, architecture_name, known_architectures, load_config,  # noqa: F401
                       register_architecture, resolve_architecture)
