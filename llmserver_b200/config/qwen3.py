"""Typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

The reference keeps no typed configuration: ``utils/architecture.py:88-107`` turns a Hugging
Face config object into positional arguments of ``Model`` and ``utils/engine.py:75-82``
re-reads the object ad hoc.  Here every size and constant the model needs is a field of one
frozen dataclass; nothing that config.json gives is written down anywhere else.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Optional, Tuple

from .errors import UnsupportedModelError

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"
SUPPORTED_ACTIVATIONS = ("silu", "swish")  # utils/layers.py:179 — both mean x * sigmoid(x)

_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads", "rms_norm_eps")


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: Optional[int]
    hidden_act: str
    sliding_window: Optional[int]
    layer_types: Tuple[str, ...]
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    extra: dict = field(default_factory=dict, compare=False)

    # ---------------------------------------------------------------- derived quantities
    @property
    def attention_scale(self) -> float:
        """utils/architecture.py:105 — head_dim ** -0.5."""
        return float(self.head_dim) ** -0.5

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def window_of(self, layer: int) -> Optional[int]:
        return self.sliding_window if self.layer_types[layer] == SLIDING_ATTENTION else None

    # ---------------------------------------------------------------- parsing
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        """Builds the configuration from config.json's keys.

        Defaults are those the reference applies when a key is absent: ``head_dim`` =
        hidden_size // num_attention_heads (utils/architecture.py:88), ``rope_theta`` from
        ``rope_parameters`` else 10000 (utils/architecture.py:23-30), ``hidden_act`` "silu"
        (utils/architecture.py:84).  Features it refuses are refused here with the same kind
        of message (utils/architecture.py:77-86), except sliding-window layers, which this
        engine runs."""
        def reject(reason):
            raise UnsupportedModelError(f"Model type {raw.get('model_type', '?')!r} is not supported: {reason}")

        missing = [key for key in _REQUIRED if raw.get(key) is None]
        if missing:
            raise UnsupportedModelError(f"config.json lacks required keys: {', '.join(missing)}")
        hidden, heads, kv_heads = int(raw["hidden_size"]), int(raw["num_attention_heads"]), int(raw["num_key_value_heads"])
        layers = int(raw["num_hidden_layers"])
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads"):
            if int(raw[key]) <= 0:
                reject(f"{key} must be positive: {raw[key]}")
        if heads % kv_heads:
            # utils/attention.py:186-187 raises this at the first forward; here it fails at load
            reject(f"num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})")
        head_dim = raw.get("head_dim") or hidden // heads
        if head_dim <= 0 or head_dim % 2:
            reject(f"head_dim must be positive and even for rotary embeddings: {head_dim}")

        scaling = raw.get("rope_scaling") or raw.get("rope_parameters") or {}
        rope_type = scaling.get("rope_type", scaling.get("type", "default"))
        if rope_type not in (None, "default"):
            reject(f"RoPE type {rope_type!r} is not supported (supported: default)")
        theta = raw.get("rope_theta")
        if theta is None:
            theta = scaling.get("rope_theta", 10000.0)
        if raw.get("partial_rotary_factor", 1.0) not in (1.0, None):
            reject("partial rotary embeddings are not implemented")
        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            if raw.get(key):
                reject(f"{key} is not implemented")
        if raw.get("attention_bias"):
            reject("attention projections with biases are not implemented")
        if raw.get("mlp_bias"):
            reject("feed-forward projections with biases are not implemented")
        activation = raw.get("hidden_act", "silu")
        if activation not in SUPPORTED_ACTIVATIONS:
            reject(f"activation {activation!r} is not supported (supported: {sorted(SUPPORTED_ACTIVATIONS)})")

        window = raw.get("sliding_window")
        types = raw.get("layer_types")
        if types is None:
            use_window = raw.get("use_sliding_window")
            if use_window and window:
                first = int(raw.get("max_window_layers", 0))
                types = [SLIDING_ATTENTION if index >= first else FULL_ATTENTION for index in range(layers)]
            else:
                types = [FULL_ATTENTION] * layers
        types = tuple(types)
        if len(types) != layers:
            reject(f"layer_types has {len(types)} entries for {layers} layers")
        unknown = sorted(set(types) - {FULL_ATTENTION, SLIDING_ATTENTION})
        if unknown:
            reject(f"unknown layer types {unknown}")
        if SLIDING_ATTENTION in types:
            if not window or int(window) <= 0:
                reject("sliding_attention layers need a positive sliding_window")
            window = int(window)
        else:
            window = None

        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        architectures = raw.get("architectures") or ["Qwen3ForCausalLM"]
        known = set(cls.__dataclass_fields__) | {"architectures", "rope_scaling", "rope_parameters",
                                                  "use_sliding_window", "max_window_layers"}
        return cls(
            vocab_size=int(raw["vocab_size"]), hidden_size=hidden, intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
            head_dim=int(head_dim), rms_norm_eps=float(raw["rms_norm_eps"]), rope_theta=float(theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=raw.get("max_position_embeddings"),
            hidden_act=activation, sliding_window=window, layer_types=types, eos_token_id=eos,
            bos_token_id=raw.get("bos_token_id"), architecture=architectures[0],
            model_type=raw.get("model_type", "qwen3"),
            extra={key: value for key, value in raw.items() if key not in known},
        )

    @classmethod
    def from_json_file(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as handle:
            return cls.from_dict(json.load(handle))

    def to_dict(self) -> dict:
        """config.json form (round-trips through ``from_dict``)."""
        out = asdict(self)
        out.pop("extra")
        out["architectures"] = [out.pop("architecture")]
        out["layer_types"] = list(self.layer_types)
        eos = list(self.eos_token_id)
        out["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        out["use_sliding_window"] = self.sliding_window is not None
        out["torch_dtype"] = "bfloat16"
        return out
