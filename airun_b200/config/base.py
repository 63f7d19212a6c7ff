"""Typed model configuration and the architecture registry.

A configuration is read from the keys of the architecture's own ``config.json``.
The registry maps the name found in ``architectures[0]`` to a pair
(configuration class, model builder); nothing else in the package knows a
model by name.  The reference resolves an architecture string to an enum the
same way and answers an unknown one with the list of those it supports
(crates/airun-core/src/config.rs:26-44, crates/airun-core/src/error.rs:24-29).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message lists every problem found."""


@dataclass(frozen=True)
class LayerSpec:
    """What one layer is made of, chosen layer by layer.

    ``mixer`` and ``feed_forward`` are names in the part registries
    (airun_b200.parts.registry); ``mixer_args`` / ``ffn_args`` are the sizes and
    constants the part is built with.
    """
    mixer: str
    mixer_args: Dict[str, Any]
    feed_forward: str
    ffn_args: Dict[str, Any]
    norm: str
    norm_args: Dict[str, Any]
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the execution order.

    ``layer`` indexes the model's layer list (the same layer may be named by
    several entries).  ``cache_from`` is None when the entry owns a cache of its
    own, or the index of an earlier entry of the order whose cache it reads
    instead of writing one.
    """
    layer: int
    cache_from: Optional[int] = None


class ModelConfig:
    """Interface every architecture's configuration offers to the engine."""

    architecture: str

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def layer_specs(self) -> List[LayerSpec]:
        raise NotImplementedError

    def execution_order(self) -> List[LayerCall]:
        return [LayerCall(i) for i in range(len(self.layer_specs()))]

    def embedding(self) -> Tuple[str, dict]:
        """(registered name, constructor arguments) of the embedding part, e.g. ("token_embedding", {"scale": 8.0})."""
        return "token_embedding", {}

    def head(self) -> Tuple[str, dict]:
        """(registered name, constructor arguments) of the output head, e.g. ("lm_head", {"soft_cap": 30.0})."""
        return "lm_head", {}


_REGISTRY: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_cls: type, builder: Callable) -> None:
    """Registers ``builder(config, dtype, device) -> Model`` under ``name``."""
    _REGISTRY[name] = (config_cls, builder)


def registered_architectures() -> List[str]:
    return sorted(_REGISTRY)


def lookup_architecture(name: str) -> Tuple[type, Callable]:
    if name not in _REGISTRY:
        raise ConfigError(
            f"architecture {name!r} is not supported; registered: "
            f"{', '.join(registered_architectures()) or '(none)'}")
    return _REGISTRY[name]


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path} not found: a model folder holds config.json and model.safetensors")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d


def architecture_name(d: Dict[str, Any]) -> str:
    archs = d.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    raise ConfigError("config.json is missing 'architectures' (a list whose first entry names the model class)")


def load_config(model_dir: str) -> ModelConfig:
    """config.json of ``model_dir`` as the typed configuration of its architecture."""
    d = read_config_json(model_dir)
    config_cls, _ = lookup_architecture(architecture_name(d))
    return config_cls.from_dict(d)
