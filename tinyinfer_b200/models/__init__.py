from .decoder import DecoderModel
from .qwen3 import Qwen3ForCausalLM

__all__ = ["DecoderModel", "Qwen3ForCausalLM"]
