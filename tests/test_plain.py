"""The plain implementation checked against closed forms (no GPU), as the reference checks its
kernels: tests/unit/test_rmsnorm.cpp:22-76, test_rope.cpp:13-67, test_softmax.cpp:22-79."""
import math

import numpy as np

import plain_qwen3 as P
from conftest import random_ids


def test_rmsnorm_closed_form():
    x = np.array([[1.0, 2.0, 3.0, 4.0]])
    y = P.rmsnorm(x, np.ones(4), 0.0)
    assert np.allclose(y, x / math.sqrt(7.5))
    assert np.allclose(P.rmsnorm(x, np.array([2.0, 0, 0, 0]), 0.0)[0, 0], 2 / math.sqrt(7.5))


def test_rope_identity_pairs_and_norms():
    x = np.random.default_rng(0).standard_normal((3, 2, 8))
    assert np.allclose(P.rope_half_split(x, [0, 0, 0], 1e4), x)
    e = np.zeros((1, 1, 8))
    e[0, 0, 0] = 1.0
    r = P.rope_half_split(e, [1], 1e4)
    assert np.isclose(r[0, 0, 0], math.cos(1.0)) and np.isclose(r[0, 0, 4], math.sin(1.0))
    y = P.rope_half_split(x, [5, 9, 200], 1e6)
    for j in range(4):
        assert np.allclose(x[..., j] ** 2 + x[..., j + 4] ** 2, y[..., j] ** 2 + y[..., j + 4] ** 2)


def test_softmax_uniform_and_stable():
    assert np.allclose(P.softmax(np.zeros(5)), 0.2)
    s = P.softmax(np.array([100.0, 101.0, 102.0]))
    assert np.isclose(s.sum(), 1.0) and np.all(np.isfinite(s))


def test_attention_window_and_groups():
    rng = np.random.default_rng(1)
    T, nh, nkv, d = 9, 4, 2, 8
    q, k, v = rng.standard_normal((T, nh, d)), rng.standard_normal((T, nkv, d)), rng.standard_normal((T, nkv, d))
    full = P.attention(q, k, v, np.arange(T))
    assert np.allclose(full[0], np.repeat(v[0], 2, axis=0))          # one key: its value
    w3 = P.attention(q, k, v, np.arange(T), window=3)
    assert np.allclose(w3[:3], full[:3]) and not np.allclose(w3[5], full[5])
    # the last token with window 3 sees exactly keys 6, 7, 8
    s = (k[6:9, 1] @ q[8, 3]) / math.sqrt(d)
    assert np.allclose(w3[8, 3], P.softmax(s) @ v[6:9, 1])


def test_forward_prefix_property_and_tied_head(plain_models):
    for name in ("A", "C"):
        cfg, w = plain_models(name, "float32")
        ids = random_ids(3, 30, cfg["vocab_size"])
        whole = P.forward(cfg, w, ids)
        assert whole.shape == (30, cfg["vocab_size"])
        assert np.allclose(P.forward(cfg, w, ids[:11]), whole[:11], atol=1e-12)   # causal
    cfg, w = plain_models("A", "float32")
    assert "lm_head.weight" not in w and cfg["tie_word_embeddings"]


def test_greedy_stops_before_the_stop_token(plain_models):
    cfg, w = plain_models("A", "float32")
    out = P.greedy_generate(cfg, w, [1, 2, 3], 6)
    assert len(out) == 6
    cut = P.greedy_generate(cfg, w, [1, 2, 3], 6, stop_ids=(out[2],))
    assert cut == out[:out.index(out[2])]
