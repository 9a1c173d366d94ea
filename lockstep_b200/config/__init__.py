"""Typed configurations and the architecture registry."""

from .registry import (architecture_name, config_from_dict, known_architectures, load_config,
                       register_architecture, unregister_architecture)
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec, own_tensors, tensor_name
from . import qwen3 as _qwen3  # registers Qwen3ForCausalLM
from .qwen3 import Qwen3Config
from . import sevipel as _sevipel  # registers Sevipel
from .sevipel import SevipelConfig
from . import malazen as _malazen  # registers Malazen
from .malazen import MalazenConfig
from . import kemirax as _kemirax  # registers Kemirax
from .kemirax import KemiraxConfig
from . import pikurax as _pikurax  # registers Pikurax
from .pikurax import PikuraxConfig

__all__ = [
    "ConfigError", "KemiraxConfig", "LayerRun", "LayerSpec", "MalazenConfig", "ModelSpec", "PartSpec", "PikuraxConfig", "Qwen3Config", "SevipelConfig",
    "architecture_name", "config_from_dict", "known_architectures", "load_config",
    "own_tensors", "register_architecture", "tensor_name", "unregister_architecture",
]
