"""The typed GPT-2 configuration, read from GPT-2's own config.json keys.

The reference reads `n_layer n_head n_embd vocab_size n_positions layer_norm_epsilon
eos_token_id` and nothing else (kelpie-models/kelpie_models/models/torch/gpt2.py:145-154); its
GPT2Config is the frozen dataclass at gpt2.py:26-42. The further keys here (`n_inner`,
`activation_function`, `scale_attn_weights`, `scale_attn_by_inverse_layer_idx`,
`tie_word_embeddings`) carry the meaning that the key has in a GPT-2 config.json; where a
file leaves one out, the value is GPT-2's documented default for that key, never a size.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, asdict

from .registry import ConfigError

ACTIVATIONS = ("gelu_new", "gelu")

_REQUIRED_INT = ("n_layer", "n_head", "n_embd", "vocab_size", "n_positions")


def _require_int(data: dict, key: str, minimum: int = 1) -> int:
    if key not in data:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    value = data[key]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {key!r} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: {key!r} must be >= {minimum}, got {value}")
    return value


def _optional_bool(data: dict, key: str, default: bool) -> bool:
    value = data.get(key, default)
    if not isinstance(value, bool):
        raise ConfigError(f"config.json: {key!r} must be true or false, got {value!r}")
    return value


def _optional_token(data: dict, key: str, vocab: int) -> int | None:
    value = data.get(key)
    if value is None:
        return None
    if isinstance(value, bool) or not isinstance(value, int) or not 0 <= value < vocab:
        raise ConfigError(f"config.json: {key!r} must be a token id in [0, {vocab}), got {value!r}")
    return value


@dataclass(frozen=True)
class GPT2Config:
    n_layer: int
    n_head: int
    n_embd: int
    vocab_size: int
    n_positions: int
    layer_norm_epsilon: float
    n_inner: int
    activation_function: str
    scale_attn_weights: bool
    scale_attn_by_inverse_layer_idx: bool
    tie_word_embeddings: bool
    eos_token_id: int | None
    bos_token_id: int | None

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def n_kv_heads(self) -> int:
        """GPT-2 has as many KV heads as query heads (reference gpt2.py:40-42)."""
        return self.n_head

    @property
    def max_seq_len(self) -> int:
        return self.n_positions

    def attention_scale(self, layer_idx: int) -> float:
        scale = self.head_dim**-0.5 if self.scale_attn_weights else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            scale /= float(layer_idx + 1)
        return scale

    @staticmethod
    def from_json(data: dict) -> "GPT2Config":
        ints = {key: _require_int(data, key) for key in _REQUIRED_INT}
        if "layer_norm_epsilon" not in data:
            raise ConfigError("config.json: required key 'layer_norm_epsilon' is missing")
        eps = data["layer_norm_epsilon"]
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps <= 0:
            raise ConfigError(f"config.json: 'layer_norm_epsilon' must be a positive number, got {eps!r}")
        if ints["n_embd"] % ints["n_head"] != 0:
            raise ConfigError(
                f"config.json: n_embd ({ints['n_embd']}) is not a multiple of n_head ({ints['n_head']})"
            )
        n_inner = data.get("n_inner")
        if n_inner is None:
            n_inner = 4 * ints["n_embd"]  # GPT-2's meaning of a null n_inner
        elif isinstance(n_inner, bool) or not isinstance(n_inner, int) or n_inner < 1:
            raise ConfigError(f"config.json: 'n_inner' must be a positive integer or null, got {n_inner!r}")
        activation = data.get("activation_function", "gelu_new")
        if activation not in ACTIVATIONS:
            raise ConfigError(
                f"config.json: activation_function {activation!r} is not supported "
                f"(supported: {', '.join(ACTIVATIONS)})"
            )
        tie = _optional_bool(data, "tie_word_embeddings", True)
        if not tie:
            raise ConfigError(
                "config.json: tie_word_embeddings=false is not supported: GPT-2's head is its "
                "token embedding (no separate lm_head tensor is read)"
            )
        vocab = ints["vocab_size"]
        return GPT2Config(
            n_layer=ints["n_layer"],
            n_head=ints["n_head"],
            n_embd=ints["n_embd"],
            vocab_size=vocab,
            n_positions=ints["n_positions"],
            layer_norm_epsilon=float(eps),
            n_inner=n_inner,
            activation_function=activation,
            scale_attn_weights=_optional_bool(data, "scale_attn_weights", True),
            scale_attn_by_inverse_layer_idx=_optional_bool(data, "scale_attn_by_inverse_layer_idx", False),
            tie_word_embeddings=tie,
            eos_token_id=_optional_token(data, "eos_token_id", vocab),
            bos_token_id=_optional_token(data, "bos_token_id", vocab),
        )

    def to_json(self) -> dict:
        out = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2"}
        out.update(asdict(self))
        return out
