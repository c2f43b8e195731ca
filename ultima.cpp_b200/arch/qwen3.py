"""Qwen3 dense as data: which parts each layer has, their constants, the tensor names.

Reference: the registry row of this architecture (src/model/arch_registry.cpp:18-19: SiLU-gated
dense feed-forward, separate Q/K/V, half-split rotary pairing, no attention gate) and the
order of one layer (src/model/qwen_block.cpp:596-814: norm, q/k/v, per-head norm, rotation,
cache write, attention, output projection, residual, norm, feed-forward, residual).
"""
from __future__ import annotations

from ..config.base import ArchitectureEntry, register_architecture
from ..config.qwen3 import Qwen3Config
from ..parts.base import ModelSpec, Run, layer, part

_NAMES = (("mixer", "self_attn."), ("feed_forward", "mlp."), ("mixer_norm", "input_layernorm."),
          ("feed_forward_norm", "post_attention_layernorm."))


def build_spec(cfg: Qwen3Config, max_positions: int | None = None) -> ModelSpec:
    max_pos = int(max_positions or cfg.max_position_embeddings)
    position = part("rotary_half_split", head_dim=cfg.head_dim, theta=cfg.rope_theta,
                    max_positions=max_pos)
    norm = part("rms", width=cfg.hidden_size, eps=cfg.rms_norm_eps)
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = part("attention", width=cfg.hidden_size, n_heads=cfg.num_attention_heads,
                     n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, qk_norm=True,
                     eps=cfg.rms_norm_eps, position=position, window=cfg.window_of_layer(i))
        ffn = part("gated_silu", width=cfg.hidden_size, inner=cfg.intermediate_size)
        layers.append(layer(part("pre_norm"), prefix=f"model.layers.{i}.", names=_NAMES, mixer=mixer,
                            feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm))
    return ModelSpec(
        width=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=max_pos,
        embedding=part("token_table", vocab_size=cfg.vocab_size, width=cfg.hidden_size),
        embedding_name="model.embed_tokens.",
        layers=tuple(layers), runs=tuple(Run(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm, final_norm_name="model.norm.",
        head=part("linear", vocab_size=cfg.vocab_size, width=cfg.hidden_size,
                  tied=cfg.tie_word_embeddings),
        head_name="lm_head.", stop_token_ids=tuple(cfg.eos_token_id))


register_architecture(ArchitectureEntry(
    name="Qwen3ForCausalLM", model_type="qwen3", supported=True,
    notes="Qwen3 dense: Q/K RMSNorm, no attention biases, gated SiLU feed-forward",
    config_cls=Qwen3Config, build_spec=build_spec))
