"""Typed configuration of the dense Qwen3 decoder, read from its config.json keys.

The reference reads the same quantities from GGUF metadata and validates them in
src/minillm/qwen3_model.cpp:9-40 (dimensions in [1, 1e6], heads divisible by kv
heads, even head size, finite positive eps and rope base, no rope scaling); the
checks here are the same ones, on config.json.  Every size comes from the file:
a missing required key is an error, not a default.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import List, Optional, Tuple

from .base import ConfigError

_LIMIT = 1_000_000


def _integer(raw: dict, key: str, default=None) -> int:
    value = raw.get(key, default)
    if value is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json key {key!r} must be an integer, got {value!r}")
    if not 1 <= value <= _LIMIT:
        raise ConfigError(f"config.json key {key!r} = {value} is outside [1, {_LIMIT}]")
    return value


def _positive_float(raw: dict, key: str, value) -> float:
    if value is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json key {key!r} must be a number, got {value!r}")
    value = float(value)
    if not math.isfinite(value) or value <= 0:
        raise ConfigError(f"config.json key {key!r} = {value} must be finite and positive")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    layer_windows: Tuple[Optional[int], ...]   # per layer: None = all keys, n = the last n keys
    eos_token_ids: Tuple[int, ...]
    stored_dtype: str

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        arch = raw.get("architectures", [None])[0]
        hidden = _integer(raw, "hidden_size")
        layers = _integer(raw, "num_hidden_layers")
        heads = _integer(raw, "num_attention_heads")
        kv_heads = _integer(raw, "num_key_value_heads", heads)
        if raw.get("head_dim") is None:
            if hidden % heads:
                raise ConfigError(f"head_dim is absent and hidden_size {hidden} is not divisible by num_attention_heads {heads}")
            head_dim = hidden // heads
        else:
            head_dim = _integer(raw, "head_dim")
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for the half-split rotation")
        inter = _integer(raw, "intermediate_size")
        vocab = _integer(raw, "vocab_size")
        max_pos = _integer(raw, "max_position_embeddings")
        eps = _positive_float(raw, "rms_norm_eps", raw.get("rms_norm_eps"))
        rope_params = raw.get("rope_parameters") if isinstance(raw.get("rope_parameters"), dict) else {}
        theta = _positive_float(raw, "rope_theta", raw.get("rope_theta", rope_params.get("rope_theta")))
        scaling = raw.get("rope_scaling")
        scaling_type = None
        if isinstance(scaling, dict):
            scaling_type = scaling.get("rope_type", scaling.get("type"))
        elif rope_params:
            scaling_type = rope_params.get("rope_type")
        if scaling_type not in (None, "none", "default"):
            raise ConfigError(f"rope scaling {scaling_type!r} is not supported (only unscaled rotation)")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias = true is not supported: the projections have no bias")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported: the feed-forward is SiLU-gated")
        windows = cls._windows(raw, layers)
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"eos_token_id {e} is outside the vocabulary of {vocab}")
        stored = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
        return cls(architecture=arch, hidden_size=hidden, num_hidden_layers=layers,
                   num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                   intermediate_size=inter, vocab_size=vocab, max_position_embeddings=max_pos,
                   rms_norm_eps=eps, rope_theta=theta,
                   tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
                   layer_windows=windows, eos_token_ids=eos_ids, stored_dtype=str(stored))

    @staticmethod
    def _windows(raw: dict, layers: int) -> Tuple[Optional[int], ...]:
        """Which layers read a window of keys.  `use_sliding_window` switches it on;
        then `layer_types` names each layer, or layers from `max_window_layers` on
        read the last `sliding_window` keys."""
        if not raw.get("use_sliding_window", False):
            return (None,) * layers
        window = raw.get("sliding_window")
        if window is None:
            return (None,) * layers
        window = _integer(raw, "sliding_window")
        kinds = raw.get("layer_types")
        if kinds is not None:
            if not isinstance(kinds, list) or len(kinds) != layers:
                raise ConfigError(f"layer_types must list {layers} layers")
            for k in kinds:
                if k not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"layer_types entry {k!r} is neither full_attention nor sliding_attention")
            return tuple(window if k == "sliding_attention" else None for k in kinds)
        first = raw.get("max_window_layers", layers)
        if isinstance(first, bool) or not isinstance(first, int) or first < 0:
            raise ConfigError(f"max_window_layers must be a non-negative integer, got {first!r}")
        return tuple(window if i >= first else None for i in range(layers))

    def to_dict(self) -> dict:
        """A config.json that parses back to this configuration."""
        windows = [w for w in self.layer_windows if w is not None]
        out = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "use_sliding_window": bool(windows),
            "torch_dtype": self.stored_dtype,
        }
        if windows:
            out["sliding_window"] = windows[0]
            out["layer_types"] = ["sliding_attention" if w is not None else "full_attention"
                                  for w in self.layer_windows]
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out

    def describe(self) -> dict:
        return asdict(self)
