"""Typed configurations and the architecture registry."""

from .registry import (  # noqa: F401
    Architecture,
    ConfigError,
    architecture_of,
    known_architectures,
    load_config,
    lookup_architecture,
    read_config_json,
    register_architecture,
    unregister_architecture,
)
from .llama import Llama3RopeScaling, LlamaConfig, read_rope_parameters  # noqa: F401
