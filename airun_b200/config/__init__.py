"""Typed configurations and the registry from architecture name to model."""
from .base import (ConfigError, LayerCall, LayerSpec, ModelConfig, architecture_name, load_config,
                   lookup_architecture, read_config_json, register_architecture, registered_architectures)
from .qwen3 import Qwen3Config


def _register_builtin() -> None:
    from ..engine.model import build_decoder
    register_architecture("Qwen3ForCausalLM", Qwen3Config, build_decoder)


_register_builtin()
