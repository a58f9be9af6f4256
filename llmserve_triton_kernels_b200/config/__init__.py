from .llama import ConfigError, LlamaConfig  # noqa: F401
from .registry import (  # noqa: F401
    Architecture,
    architecture_of,
    get_architecture,
    known_architectures,
    read_config,
    register_architecture,
    unregister_architecture,
)
