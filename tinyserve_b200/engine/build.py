"""From a configuration to a model made of parts."""
from __future__ import annotations

from ..config.model_config import ModelConfig
from ..parts.model import DecoderModel


def build_model(config: ModelConfig) -> DecoderModel:
    return DecoderModel(config.model_spec())
