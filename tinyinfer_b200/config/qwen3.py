"""Typed configuration of the Qwen3 dense decoder, read from the keys of its own config.json.

Which keys exist and what they default to follows the reference's model code
(tinyinfer/models/qwen3.py:39-48 rope_theta, :58-61 heads and head_dim, :69 attention_bias,
:73-74 rms_norm_eps for all norms, :148-150 intermediate_size, :228 vocab_size,
:271-272 tie_word_embeddings; tinyinfer/config.py:39-40 max_position_embeddings).
The sliding-window keys (sliding_window, use_sliding_window, max_window_layers, layer_types)
are the ones a Qwen3 config.json carries; the reference never reads them, so its models are the
case without a window.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import List, Optional

from .specs import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                    TensorNames, default_execution)

_REQUIRED = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "intermediate_size", "rms_norm_eps", "max_position_embeddings")


@dataclass
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    rms_norm_eps: float
    max_position_embeddings: int
    head_dim: Optional[int] = None            # falls back to hidden_size // num_attention_heads
    rope_theta: float = 10000.0
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_window_layers: Optional[int] = None
    layer_types: Optional[List[str]] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    model_type: str = "qwen3"
    architectures: List[str] = field(default_factory=lambda: ["Qwen3ForCausalLM"])

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, data: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in data]
        if missing:
            raise ValueError(f"config.json lacks required keys: {missing}")
        d = dict(data)
        if "rope_theta" not in d:
            scaling = d.get("rope_scaling")
            if isinstance(scaling, dict) and "rope_theta" in scaling:
                d["rope_theta"] = scaling["rope_theta"]
        scaling = d.get("rope_scaling")
        if isinstance(scaling, dict):
            kind = scaling.get("rope_type", scaling.get("type", "default"))
            if kind not in ("default", None):
                raise ValueError(f"rope_scaling of type {kind!r} is not supported: keys are cached "
                                 "after the rotation, so angles must not depend on the final length")
        if "dtype" in d and "torch_dtype" not in d:
            d["torch_dtype"] = d["dtype"]
        eos = d.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            d["eos_token_id"] = eos[0] if eos else None
        known = {f for f in cls.__dataclass_fields__}
        cfg = cls(**{k: v for k, v in d.items() if k in known})
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = asdict(self)
        d["head_dim"] = self.resolved_head_dim
        return {k: v for k, v in d.items() if v is not None}

    # ------------------------------------------------------------------ checks
    @property
    def resolved_head_dim(self) -> int:
        return int(self.head_dim) if self.head_dim else self.hidden_size // self.num_attention_heads

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "intermediate_size", "max_position_embeddings"):
            if int(getattr(self, key)) <= 0:
                raise ValueError(f"{key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads "
                             f"({self.num_attention_heads} vs {self.num_key_value_heads})")
        if self.resolved_head_dim % 2:
            raise ValueError(f"head_dim must be even for the rotation, got {self.resolved_head_dim}")
        if not self.rms_norm_eps > 0:
            raise ValueError("rms_norm_eps must be positive")
        if self.hidden_act != "silu":
            raise ValueError(f"hidden_act {self.hidden_act!r} is not supported (silu only)")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ValueError("layer_types must name every layer")
            bad = set(self.layer_types) - {"full_attention", "sliding_attention"}
            if bad:
                raise ValueError(f"unknown layer_types {sorted(bad)}")
            if "sliding_attention" in self.layer_types and not self.sliding_window:
                raise ValueError("layer_types names sliding_attention but sliding_window is unset")
        if self.sliding_window is not None and int(self.sliding_window) <= 0:
            raise ValueError("sliding_window must be positive")

    # ------------------------------------------------------------------ layers
    def layer_windows(self) -> List[Optional[int]]:
        n = self.num_hidden_layers
        if self.layer_types is not None:
            return [int(self.sliding_window) if t == "sliding_attention" else None
                    for t in self.layer_types]
        if self.use_sliding_window and self.sliding_window is not None:
            first = n if self.max_window_layers is None else int(self.max_window_layers)
            return [int(self.sliding_window) if i >= first else None for i in range(n)]
        return [None] * n

    def model_spec(self) -> ModelSpec:
        d = self.resolved_head_dim
        eps = float(self.rms_norm_eps)
        position = PositionSpec(kind="rope", theta=float(self.rope_theta), rotary_dim=d)
        layers = []
        for window in self.layer_windows():
            mixer = AttentionSpec(
                hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads, head_dim=d, scale=float(d) ** -0.5,
                position=position, qk_norm=NormSpec(size=d, eps=eps),
                bias=bool(self.attention_bias), window=window)
            ffn = GatedMLPSpec(hidden_size=self.hidden_size,
                               intermediate_size=self.intermediate_size, activation=self.hidden_act)
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn,
                                    mixer_norm=NormSpec(self.hidden_size, eps),
                                    feed_forward_norm=NormSpec(self.hidden_size, eps)))
        return ModelSpec(
            architecture=self.architectures[0], vocab_size=self.vocab_size,
            hidden_size=self.hidden_size, layers=tuple(layers),
            execution=default_execution(self.num_hidden_layers),
            final_norm=NormSpec(self.hidden_size, eps),
            tie_embeddings=bool(self.tie_word_embeddings),
            max_positions=self.max_position_embeddings, names=TensorNames())
