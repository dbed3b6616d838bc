"""The one registry from an architecture's name to its configuration class.

``config.json["architectures"][0]`` selects the entry; everything that loads a
model folder (the Python entry point, the command line, trace replay, the bench)
goes through ``load_model_config``.  tinyserve dispatches on ``model_type`` with
``if`` switches inside one Model class (serve.py:70, 824, 831, 1305); here an
architecture is a configuration class whose ``model_spec()`` names the parts.
"""
from __future__ import annotations

import json
import os

from .model_config import ConfigError, ModelConfig, Qwen3Config

ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    """Add (or replace) an architecture.  ``config_cls`` is a ModelConfig subclass."""
    if not (isinstance(config_cls, type) and issubclass(config_cls, ModelConfig)):
        raise TypeError("config_cls must be a ModelConfig subclass")
    ARCHITECTURES[name] = config_cls


def architecture_of(raw: dict) -> str:
    names = raw.get("architectures")
    if not names or not isinstance(names, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list")
    return names[0]


def config_from_dict(raw: dict) -> ModelConfig:
    name = architecture_of(raw)
    if name not in ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not registered; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[name].from_dict(raw)


def load_model_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir!r} holds no config.json")
    with open(path) as fh:
        return config_from_dict(json.load(fh))


register_architecture(Qwen3Config.architecture, Qwen3Config)
