from .engine_config import EngineConfig, parse_dtype
from .registry import (Architecture, architecture_of, known_architectures, known_presets, load_config,
                       lookup_architecture, preset_config, register_architecture)
from .specs import (AttentionSpec, ExecStep, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                    PositionSpec, TensorNames, default_execution)
from .qwen3 import Qwen3Config

__all__ = [
    "EngineConfig", "parse_dtype", "Architecture", "architecture_of", "known_architectures",
    "known_presets", "load_config", "lookup_architecture", "preset_config", "register_architecture", "AttentionSpec", "ExecStep",
    "GatedMLPSpec", "LayerSpec", "ModelSpec", "NormSpec", "PositionSpec", "TensorNames",
    "default_execution", "Qwen3Config",
]
