"""A plain, slow restatement of the Qwen3 dense decoder, used only as the tests' oracle.

Whole sequences, no cache, one function for each part, float64 by default.  It shares no
code with the package: it reads ``config.json`` as a dict and ``model.safetensors`` with its
own few lines.  Every function cites the place in the reference (tattooinmtl/Ultima.cpp,
paths inside that project) whose arithmetic it restates.  tests/golden/ holds the logits
of the reference's own model code on two tiny random models, which this file is compared
with in tests/test_plain_vs_reference.py.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ---------------------------------------------------------------------------------------
# reading a model folder (independent of the package's loader)
# ---------------------------------------------------------------------------------------
def read_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    path = os.path.join(model_dir, "model.safetensors")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    header.pop("__metadata__", None)
    weights = {}
    for name, e in header.items():
        b, end = e["data_offsets"]
        raw = data[b:end]
        if e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif e["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"plain reader: dtype {e['dtype']} of {name}")
        weights[name] = a.reshape(e["shape"])
    return cfg, weights


# ---------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------
def embed(table, ids):
    """x_t = E[id_t, :], no scaling.  src/model/qwen_model.cpp:145-157."""
    ids = np.asarray(ids)
    if ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token id out of range")          # qwen_model.cpp:147-152
    return table[ids]


def rmsnorm(x, w, eps):
    """y = x * w / sqrt(mean(x^2) + eps) over the last axis.  src/kernels/rmsnorm.cpp:10-17."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x * w * (1.0 / np.sqrt(ms + eps))


def linear(x, w):
    """y[t, m] = sum_k W[m, k] x[t, k], row-major [out, in].  src/kernels/matvec_f32_f32.cpp:8-18."""
    return x @ w.T


def rope_half_split(x, positions, theta):
    """Rotation of the pairs (x[j], x[j + half]) by pos * theta^(-2j/d).
    x: [T, heads, d].  src/kernels/rope.cpp:17-52 (pairing :42-43, angle :34-38)."""
    d = x.shape[-1]
    half = d // 2
    j = np.arange(half, dtype=np.float64)
    inv = 1.0 / np.power(float(theta), 2.0 * j / d)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]      # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)


def softmax(s):
    """max-shift, exp, sum, scale.  src/kernels/softmax.cpp:9-29."""
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def attention(q, k, v, positions, window=None):
    """Grouped-query attention of one sequence over itself.

    q: [T, nh, d], k, v: [T, nkv, d] (k after norm and rotation), positions: [T] absolute.
    Query head h reads KV head h // (nh/nkv); the token at position p sees keys at
    positions (p - window, p] (all positions <= p without a window); scale 1/sqrt(d).
    src/model/qwen_block.cpp:94-135 (group mapping :106-110, scores :114-120, weighted sum
    :127-133), window :742-745, scale :732-734.
    """
    T, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(d)
    out = np.zeros_like(q)
    for t in range(T):
        n_keys = t + 1
        begin = 0
        if window is not None and n_keys > window:
            begin = n_keys - window
        for h in range(nh):
            g = h // group
            s = (k[begin:n_keys, g, :] @ q[t, h, :]) * scale
            w = softmax(s)
            out[t, h, :] = w @ v[begin:n_keys, g, :]
    return out


def swiglu(gate, up):
    """a = gate / (1 + exp(-gate)) * up.  src/kernels/elementwise.cpp:62-68."""
    return gate / (1.0 + np.exp(-gate)) * up


def attention_part(h, w, prefix, cfg, positions, window):
    """Projections, per-head norm of q and k, rotation, attention, output projection.
    src/model/qwen_block.cpp:682-690 (q, k, v), :713-718 (per-head norm, same eps),
    :719-723 (rotation after the norm), :736-751 (attention), :775-778 (output)."""
    T = h.shape[0]
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg.get("rms_norm_eps", 1e-6)
    q = linear(h, w[prefix + "q_proj.weight"]).reshape(T, nh, d)
    k = linear(h, w[prefix + "k_proj.weight"]).reshape(T, nkv, d)
    v = linear(h, w[prefix + "v_proj.weight"]).reshape(T, nkv, d)
    q = rmsnorm(q, w[prefix + "q_norm.weight"], eps)
    k = rmsnorm(k, w[prefix + "k_norm.weight"], eps)
    q = rope_half_split(q, positions, cfg["rope_theta"])
    k = rope_half_split(k, positions, cfg["rope_theta"])
    o = attention(q, k, v, positions, window).reshape(T, nh * d)
    return linear(o, w[prefix + "o_proj.weight"])


def mlp_part(h, w, prefix):
    """down(silu(gate(h)) * up(h)).  src/model/qwen_block.cpp:165-182."""
    a = swiglu(linear(h, w[prefix + "gate_proj.weight"]), linear(h, w[prefix + "up_proj.weight"]))
    return linear(a, w[prefix + "down_proj.weight"])


def layer_window(cfg, i):
    types = cfg.get("layer_types")
    if types and cfg.get("sliding_window") and cfg.get("use_sliding_window", True) is not False:
        if types[i] == "sliding_attention":
            return int(cfg["sliding_window"])
    return None


def block(x, w, i, cfg, positions):
    """Pre-norm block: x += attn(norm(x)); x += mlp(norm(x)).  src/model/qwen_block.cpp:621-628,
    :782-792, :811-812."""
    p = f"model.layers.{i}."
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_part(h, w, p + "self_attn.", cfg, positions, layer_window(cfg, i))
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    return x + mlp_part(h, w, p + "mlp.")


def forward(cfg, w, ids):
    """Logits [len(ids), vocab] of one whole sequence.  src/model/qwen_model.cpp:136-210
    (embedding :145-157, layers :174-180, final norm :183-188, head :189-202, tied head
    when the file has no separate one, src/model/qwen_tensor_slots.cpp:150-158)."""
    positions = np.arange(len(ids))
    x = embed(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        x = block(x, w, i, cfg, positions)
    h = rmsnorm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return linear(h, head)


# ---------------------------------------------------------------------------------------
# sampling (the package's own rule for the random draw, restated)
# ---------------------------------------------------------------------------------------
def argmax_first(logits):
    """First maximum wins.  src/sampler/sampler.cpp:220-228."""
    best, bv = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > bv:
            best, bv = i, logits[i]
    return best


def greedy_generate(cfg, w, prompt, n_new, stop_ids=()):
    """Prefill, then sample / stop check / feed.  The stop token is neither emitted nor fed.
    apps/ultima-cli/main.cpp:652-686."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        nxt = argmax_first(forward(cfg, w, ids)[-1])
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
