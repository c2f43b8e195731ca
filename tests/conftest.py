"""Shared pieces of the tests: the import path, the gpu mark, the tiny configurations and
model folders made in temporary folders."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    # all tests together take a few minutes; a session that has not ended after 25 dumps every
    # thread's stack and exits, so a kernel that stopped making progress cannot hold a GPU for hours
    import faulthandler
    faulthandler.dump_traceback_later(1500, exit=True)


def pytest_unconfigure(config):
    import faulthandler
    faulthandler.cancel_dump_traceback_later()


# Three tiny configurations that differ in every size and option: layers, width, heads and
# groups (group 2, multi-query, group 2 of 3 kv heads), head size (16 / 32 / 48), Q width equal
# to or different from the width, inner size (none a multiple of 128), vocabulary (none a
# power of two but the first), rotary base, eps, tied or separate head, context, window.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=512, hidden_size=64,
              intermediate_size=192, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=128,
              tie_word_embeddings=True, hidden_act="silu")
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=96,
              intermediate_size=320, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
              head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=256,
              tie_word_embeddings=False, hidden_act="silu")
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=777, hidden_size=80,
              intermediate_size=176, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3,
              head_dim=48, rms_norm_eps=3e-6, rope_theta=500000.0, max_position_embeddings=512,
              tie_word_embeddings=False, hidden_act="silu", use_sliding_window=True, sliding_window=20,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"])
# two more with the head sizes the TMA-fed and tcgen05 attention kernels are built for (64, 128)
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=300, hidden_size=128,
              intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512,
              tie_word_embeddings=True, hidden_act="silu", use_sliding_window=True, sliding_window=40,
              layer_types=["full_attention", "sliding_attention"])
TINY_E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=401, hidden_size=192,
              intermediate_size=448, num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1,
              head_dim=128, rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=512,
              tie_word_embeddings=False, hidden_act="silu")
# and one whose sizes fit none of the tensor-core kernels: rows of 100 values (not a multiple of 8),
# a head size that is no multiple of 16, an inner size and a vocabulary that are odd
TINY_F = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=257, hidden_size=100,
              intermediate_size=131, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
              head_dim=24, rms_norm_eps=2e-6, rope_theta=50000.0, max_position_embeddings=256,
              tie_word_embeddings=False, hidden_act="silu")
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}


def make_model_dir(tmp, name: str, dtype: str, seed: int = 7) -> str:
    import ultima_b200 as u
    cfg = u.config_from_dict(TINY[name])
    d = os.path.join(str(tmp), f"tiny_{name}_{dtype}")
    if not os.path.isdir(d):
        u.write_random_model(d, cfg, seed, dtype)
    return d


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name, dtype -> model folder (written once a session, in a temporary folder)."""
    base = tmp_path_factory.mktemp("models")
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = make_model_dir(base, name, dtype)
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name, dtype -> (config dict, float64 weights) as the plain implementation reads them."""
    import plain_qwen3 as P
    got = {}

    def get(name, dtype):
        if (name, dtype) not in got:
            got[(name, dtype)] = P.read_folder(model_dirs(name, dtype))
        return got[(name, dtype)]
    return get


def random_ids(seed: int, n: int, vocab: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


# Error bounds of the comparisons with the plain (float64) implementation, relative to the
# largest logit of the reference.  float32: sums of a few hundred float32 products and the
# float32 rotation tables.  bfloat16: activations rounded to 8 bits of mantissa between
# layers; the bound is a multiple of 2^-8 that grows with the number of layers.
def close_enough(got, ref, dtype: str, layers: int = 4):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite logits"
    scale = max(1.0, float(np.abs(ref).max()))
    err = float(np.abs(got - ref).max())
    bound = 2e-5 * scale if dtype == "float32" else (2.0 ** -8) * (2 + layers) * scale
    return err, bound
