"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
import ultima_b200 as u
from ultima_b200.config import (ConfigError, Qwen3Config, config_from_dict, find_architecture,
                                known_architectures, register_architecture, ArchitectureEntry)


def test_reads_every_size_from_its_keys():
    c = config_from_dict(TINY_B)
    assert isinstance(c, Qwen3Config)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (1000, 96, 320, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (8, 1, 32)
    assert c.q_width == 256 and c.kv_width == 32 and c.q_width != c.hidden_size
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.sliding_window is None and set(c.layer_types) == {"full_attention"}


def test_head_dim_falls_back_to_width_over_heads():
    d = dict(TINY_A)
    del d["head_dim"]
    assert config_from_dict(d).head_dim == 64 // 4
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="not divisible"):
        config_from_dict(d)


def test_kv_heads_default_to_heads_and_must_divide():
    d = dict(TINY_A)
    del d["num_key_value_heads"]
    assert config_from_dict(d).num_key_value_heads == 4
    d["num_key_value_heads"] = 3
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict(d)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "rope_theta", "max_position_embeddings"])
def test_missing_required_key(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_window_needs_window_and_pattern():
    c = config_from_dict(TINY_C)
    assert c.sliding_window == 20
    assert [c.window_of_layer(i) for i in range(4)] == [20, None, 20, None]
    d = dict(TINY_C)
    d["layer_types"] = d["layer_types"][:3]
    with pytest.raises(ConfigError, match="layer_types"):
        config_from_dict(d)
    d = dict(TINY_C)
    del d["layer_types"]
    with pytest.raises(ConfigError, match="layer_types"):
        config_from_dict(d)
    d = dict(TINY_C)
    d["sliding_window"] = None
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(d)
    # a window that is switched off is no window
    d = dict(TINY_C)
    d["use_sliding_window"] = False
    assert config_from_dict(d).sliding_window is None


def test_rejects_what_the_model_does_not_apply():
    for key, val, pat in (("rope_scaling", {"rope_type": "yarn", "factor": 4.0}, "rope_scaling"),
                          ("hidden_act", "gelu", "hidden_act"), ("attention_bias", True, "attention_bias"),
                          ("head_dim", 15, "even")):
        d = dict(TINY_A)
        d[key] = val
        with pytest.raises(ConfigError, match=pat):
            config_from_dict(d)


def test_round_trip_through_config_json(tmp_path):
    for d in (TINY_A, TINY_B, TINY_C):
        c = config_from_dict(d)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert u.config_from_dir(str(tmp_path)) == c


def test_registry_unknown_and_unsupported_are_two_errors():
    with pytest.raises(ConfigError, match="unknown architecture"):
        find_architecture("NoSuchModel")
    register_architecture(ArchitectureEntry("ToyUnsupportedLM", "toy_unsupported", False, "a reason"))
    with pytest.raises(ConfigError, match="recognized but not runnable: a reason"):
        find_architecture("ToyUnsupportedLM")
    assert "Qwen3ForCausalLM" in [e.name for e in known_architectures()]
    assert find_architecture("qwen3") is find_architecture("Qwen3ForCausalLM")
    d = dict(TINY_A)
    d["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict(d)


def test_model_description_is_data():
    spec = u.model_spec_for(config_from_dict(TINY_C))
    assert len(spec.layers) == 4 and [r.layer for r in spec.runs] == [0, 1, 2, 3]
    assert [L.part("mixer").get("window") for L in spec.layers] == [20, None, 20, None]
    assert spec.layers[0].part("mixer").get("head_dim") == 48 and spec.layers[0].part("feed_forward").get("inner") == 176
    assert spec.layers[0].roles() == {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm",
                                      "feed_forward": "feed_forward"}
    names = {s.name: s.shape for s in spec.weight_specs()}
    assert names["model.layers.3.self_attn.q_proj.weight"] == (6 * 48, 80)
    assert names["model.layers.0.self_attn.k_norm.weight"] == (48,)
    assert names["lm_head.weight"] == (777, 80)
    tied = u.model_spec_for(config_from_dict(TINY_A))
    assert "lm_head.weight" not in {s.name for s in tied.weight_specs()}


def test_stop_tokens_come_from_both_json_files(tmp_path):
    d = dict(TINY_A, eos_token_id=7)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(d, f)
    assert u.config_from_dir(str(tmp_path)).eos_token_id == (7,)
    with open(tmp_path / "generation_config.json", "w") as f:
        json.dump({"eos_token_id": [9, 7, 11], "temperature": 0.6}, f)
    cfg = u.config_from_dir(str(tmp_path))
    assert cfg.eos_token_id == (7, 9, 11)
    assert u.model_spec_for(cfg).stop_token_ids == (7, 9, 11)
    with open(tmp_path / "generation_config.json", "w") as f:
        json.dump({"eos_token_id": "x"}, f)
    with pytest.raises(ConfigError, match="eos_token_id"):
        u.config_from_dir(str(tmp_path))


def test_an_architecture_enters_the_table_only_with_the_whole_protocol():
    """What the engine asks of a configuration class and of build_spec is checked at registration."""
    from dataclasses import dataclass
    from ultima_b200.config import ArchitectureConfig

    @dataclass(frozen=True)
    class NoToDict:
        architecture: str = "ToyLM"
        max_position_embeddings: int = 8
        torch_dtype: str = "float32"

        @classmethod
        def from_dict(cls, d):
            return cls()

    with pytest.raises(ConfigError, match="lacks to_dict"):
        register_architecture(ArchitectureEntry("ToyLM", "toy_lm", True, "", NoToDict, lambda c, max_positions=None: None))

    @dataclass(frozen=True)
    class Whole(NoToDict):
        def to_dict(self):
            return {}

    with pytest.raises(ConfigError, match="build_spec must be callable as"):
        register_architecture(ArchitectureEntry("ToyLM", "toy_lm", True, "", Whole, lambda c: None))
    assert isinstance(Whole(), ArchitectureConfig) and isinstance(config_from_dict(TINY_A), ArchitectureConfig)
    with pytest.raises(ConfigError, match="unknown architecture"):
        find_architecture("ToyLM")                         # neither attempt left anything in the table


def test_a_layer_names_its_parts_by_the_roles_of_its_arrangement():
    from ultima_b200.parts import layer, part
    norm = part("rms", width=8, eps=1e-6)
    ffn = part("gated_silu", width=8, inner=16)
    att = part("attention", width=8, n_heads=1, n_kv_heads=1, head_dim=8, qk_norm=False, eps=1e-6, position=None)
    L = layer(part("pre_norm"), prefix="x.", names={"mixer": "attn."}, mixer=att, feed_forward=ffn, mixer_norm=norm,
              feed_forward_norm=norm)
    assert L.name_of("mixer") == "x.attn." and L.name_of("feed_forward") == "x.feed_forward."
    assert L.part("feed_forward") == ffn and list(L.roles()) == ["mixer_norm", "mixer", "feed_forward_norm", "feed_forward"]
    with pytest.raises(KeyError, match="needs a part in the role 'mixer_norm'"):
        layer(part("pre_norm"), mixer=att, feed_forward=ffn, feed_forward_norm=norm)
    with pytest.raises(KeyError, match="has no role 'gate'"):
        layer(part("pre_norm"), mixer=att, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm, gate=norm)
    with pytest.raises(KeyError, match="has no part in the role 'gate'"):
        L.part("gate")
    with pytest.raises(KeyError, match="no arrangement named 'sandwich'"):
        layer(part("sandwich"), mixer=att)
