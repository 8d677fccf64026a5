"""Models are built from a `ModelSpec`; an architecture is a function from its
config.json to a spec (see `vosti_b200.config`), so adding one adds no model class."""
from typing import Dict

from ..config.schema import ModelSpec
from ..weights.loader import WeightSpec
from .decoder import DecoderModel


def build_model(spec: ModelSpec) -> DecoderModel:
    return DecoderModel(spec)


def expected_weights(spec: ModelSpec) -> Dict[str, WeightSpec]:
    return DecoderModel(spec).expected_weights()


__all__ = ["DecoderModel", "build_model", "expected_weights"]
