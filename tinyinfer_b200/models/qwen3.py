"""Qwen3 dense: the architecture this engine serves. The model is the generic decoder built from
``Qwen3Config.model_spec()``; this file only ties the name in config.json to it."""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from .decoder import DecoderModel


class Qwen3ForCausalLM(DecoderModel):
    def __init__(self, config: Qwen3Config, dtype, device):
        super().__init__(config.model_spec(), dtype, device)
        self.config = config


register_architecture("Qwen3ForCausalLM", Qwen3Config, Qwen3ForCausalLM)
