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


# Sizes of the Qwen3 family that the benchmarks run with random weights.
PRESETS = {
    "tiny": dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=16, intermediate_size=128, rms_norm_eps=1e-6,
                 rope_theta=10000.0, tie_word_embeddings=True, max_position_embeddings=512),
    "1.7b": dict(vocab_size=151936, hidden_size=2048, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, intermediate_size=6144, rms_norm_eps=1e-6,
                 rope_theta=1000000.0, tie_word_embeddings=True, max_position_embeddings=40960),
    "8b": dict(vocab_size=151936, hidden_size=4096, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=12288, rms_norm_eps=1e-6,
               rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=40960),
    "32b": dict(vocab_size=151936, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, head_dim=128, intermediate_size=25600, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=40960),
}

register_architecture("Qwen3ForCausalLM", Qwen3Config, Qwen3ForCausalLM, presets=PRESETS)
