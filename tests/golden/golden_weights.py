"""Weights for the golden comparison, from integer arithmetic only, so that the script that
ran the reference's code and the test that reads its outputs make the same numbers on any
machine and with any library version."""
import numpy as np

CONFIGS = {
    "A": dict(architectures=["Qwen3ForCausalLM"], vocab_size=512, hidden_size=64, intermediate_size=192,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=True),
    "B": dict(architectures=["Qwen3ForCausalLM"], vocab_size=1000, hidden_size=96, intermediate_size=320,
              num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1, head_dim=32,
              rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=256, tie_word_embeddings=False),
    # a window of 4 positions on the first and the last of three layers (the reference's keys
    # attention.sliding_window and attention.sliding_window_pattern, src/model/qwen_config.cpp:229-253)
    "C": dict(architectures=["Qwen3ForCausalLM"], vocab_size=300, hidden_size=48, intermediate_size=80,
              num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=16,
              rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=64, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=4,
              layer_types=["sliding_attention", "full_attention", "sliding_attention"]),
}
PROMPTS = {"A": [(37 * i * i + 11 * i + 5) % 512 for i in range(11)],
           "B": [(91 * i * i + 7 * i + 3) % 1000 for i in range(40)],
           "C": [(53 * i * i + 17 * i + 2) % 300 for i in range(16)]}
KEPT = {"A": list(range(11)), "B": [0, 1, 31, 32, 39], "C": list(range(16))}       # positions whose logits are stored


def _uniform(n: int, salt: int) -> np.ndarray:
    """n numbers in [-1, 1) from a 64-bit mixing function of (salt, index)."""
    i = np.arange(n, dtype=np.uint64) + np.uint64((salt * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)
    with np.errstate(over="ignore"):
        z = i + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(40)).astype(np.float64) / float(1 << 23) - 1.0)


def tensor_list(cfg: dict):
    """(name, shape, kind) in the order the harness reads them."""
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    out = [("model.embed_tokens.weight", (V, H), "m")]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (H,), "v"),
                (p + "self_attn.q_proj.weight", (nh * hd, H), "m"), (p + "self_attn.k_proj.weight", (nkv * hd, H), "m"),
                (p + "self_attn.v_proj.weight", (nkv * hd, H), "m"), (p + "self_attn.q_norm.weight", (hd,), "v"),
                (p + "self_attn.k_norm.weight", (hd,), "v"), (p + "self_attn.o_proj.weight", (H, nh * hd), "m"),
                (p + "post_attention_layernorm.weight", (H,), "v"),
                (p + "mlp.gate_proj.weight", (F, H), "m"), (p + "mlp.up_proj.weight", (F, H), "m"),
                (p + "mlp.down_proj.weight", (H, F), "m")]
    out.append(("model.norm.weight", (H,), "v"))
    if not cfg["tie_word_embeddings"]:
        out.append(("lm_head.weight", (V, H), "m"))
    return out


def weights(cfg: dict) -> dict:
    """name -> float32 array: matrices uniform with standard deviation 0.05, norm weights 1 +
    uniform with standard deviation 0.1 (larger than a checkpoint's, so that logits are not flat)."""
    out = {}
    for salt, (name, shape, kind) in enumerate(tensor_list(cfg)):
        n = int(np.prod(shape))
        u = _uniform(n, salt + 1)
        a = u * (0.05 * 3 ** 0.5) if kind == "m" else 1.0 + u * (0.1 * 3 ** 0.5)
        out[name] = a.astype(np.float32).reshape(shape)
    return out
