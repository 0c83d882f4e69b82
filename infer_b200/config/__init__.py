from .registry import (Architecture, ConfigError, architecture_of, get_architecture, load_config, parse_config,  # noqa: F401
                       register_architecture, registered_architectures, unregister_architecture)
from .specs import LayerCall, LayerSpec, ModelSpec, PartSpec  # noqa: F401
