from .schema import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (architecture_of, known_architectures, model_spec_from_config,
                       model_spec_from_dir, read_config_json, register_architecture)
from . import qwen3 as _qwen3
from .qwen3 import Qwen3Config

register_architecture(_qwen3.ARCHITECTURE, _qwen3.spec_from_config, replace=True)

__all__ = [
    "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
    "architecture_of", "known_architectures", "model_spec_from_config", "model_spec_from_dir",
    "read_config_json", "register_architecture",
]
