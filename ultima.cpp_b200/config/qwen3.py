"""Qwen3 dense: the typed configuration, read from the architecture's own config.json keys.

Keys and rules follow the reference's metadata parser (src/model/qwen_config.cpp:49-349):
required sizes (:64-84), head_dim from an explicit key else hidden/heads (:118-131), the
derived projection widths (:132-133), the norms' eps (:136-138), the rotary base (:147),
and the sliding window that engages only when both the window and the per-layer pattern
are present (:229-253).  Fixed by the reference's registry row for this architecture
(src/model/arch_registry.cpp:18-19): SiLU-gated feed-forward, separate Q/K/V without
biases, half-split rotary pairing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import ConfigError

FULL = "full_attention"
SLIDING = "sliding_attention"


def _need_int(d: dict, key: str, minimum: int = 1) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing required key '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


def _need_float(d: dict, key: str) -> float:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing required key '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


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
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    sliding_window: Optional[int] = None
    layer_types: tuple = ()          # one of FULL / SLIDING for each layer
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"

    # ---- derived -----------------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def window_of_layer(self, i: int) -> Optional[int]:
        return self.sliding_window if self.layer_types[i] == SLIDING else None

    # ---- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        vocab = _need_int(d, "vocab_size")
        hidden = _need_int(d, "hidden_size")
        inter = _need_int(d, "intermediate_size")
        layers = _need_int(d, "num_hidden_layers")
        heads = _need_int(d, "num_attention_heads")
        kv_heads = heads
        if d.get("num_key_value_heads") is not None:
            kv_heads = _need_int(d, "num_key_value_heads")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        if d.get("head_dim") is not None:
            head_dim = _need_int(d, "head_dim")
        else:
            if hidden % heads != 0:
                raise ConfigError(f"config.json: hidden_size {hidden} not divisible by "
                                  f"num_attention_heads {heads} and no 'head_dim' given")
            head_dim = hidden // heads
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even (rotary pairs)")
        eps = float(d["rms_norm_eps"]) if d.get("rms_norm_eps") is not None else 1e-6
        if not (eps > 0):
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, got {eps}")
        theta = _need_float(d, "rope_theta")
        if not (theta > 0):
            raise ConfigError(f"config.json: rope_theta must be > 0, got {theta}")
        max_pos = _need_int(d, "max_position_embeddings")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: 'rope_scaling' is set; scaled rotary embeddings are not "
                              "applied by this model (the reference parses them and applies none)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act must be 'silu' for this architecture, got {act!r}")
        if d.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias must be false for this architecture")
        tie = bool(d.get("tie_word_embeddings", False))

        # Sliding window: engages only with a window AND a per-layer pattern.
        window = None
        types = (FULL,) * layers
        raw_types = d.get("layer_types")
        raw_window = d.get("sliding_window")
        use = d.get("use_sliding_window", None)
        if raw_types is not None:
            if not isinstance(raw_types, list) or len(raw_types) != layers:
                n = len(raw_types) if isinstance(raw_types, list) else "no"
                raise ConfigError(f"config.json: 'layer_types' has {n} entries but the model has "
                                  f"{layers} layers")
            for t in raw_types:
                if t not in (FULL, SLIDING):
                    raise ConfigError(f"config.json: unknown layer type {t!r} in 'layer_types'")
            wants = any(t == SLIDING for t in raw_types) and use is not False
            if wants:
                if raw_window is None:
                    raise ConfigError("config.json: 'layer_types' names sliding layers but "
                                      "'sliding_window' is not set")
                window = _need_int(d, "sliding_window")
                types = tuple(raw_types)
        elif use:
            raise ConfigError("config.json: 'use_sliding_window' is true but 'layer_types' is "
                              "missing; a window without a per-layer pattern is not applied")

        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError(f"config.json: unsupported torch_dtype {dtype!r}")
        eos = d.get("eos_token_id", ())
        if eos is None:
            eos = ()
        if isinstance(eos, int):
            eos = (eos,)
        eos = tuple(int(e) for e in eos)
        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                   num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=eps,
                   rope_theta=theta, max_position_embeddings=max_pos,
                   tie_word_embeddings=tie, sliding_window=window, layer_types=types,
                   torch_dtype=dtype, eos_token_id=eos)

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        out = {
            "architectures": [self.architecture], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu",
            "attention_bias": False, "rope_scaling": None, "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            out["use_sliding_window"] = True
            out["sliding_window"] = self.sliding_window
            out["layer_types"] = list(self.layer_types)
        else:
            out["use_sliding_window"] = False
            out["sliding_window"] = None
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
