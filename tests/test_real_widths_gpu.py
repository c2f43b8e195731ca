"""The plain implementation as the oracle at the layer widths of a real checkpoint: width 4096, 32 query
and 8 KV heads of 128, inner width 12288 (Qwen3-8B's), two layers, and a vocabulary cut to 2,048 so that
float64 numpy can hold the model.  The engine's weights are drawn on the device; the oracle's are drawn
again on the host by the tests' own copy of the generator, so nothing of the package stands between the
seed and the oracle.  Whole, the last 32 tokens one by one, and a batch of unequal lengths whose shorter
requests end earlier, in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

from conftest import close_enough

pytestmark = pytest.mark.gpu

SIZES = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=2048, hidden_size=4096,
             intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
             head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=1024,
             tie_word_embeddings=False, hidden_act="silu")
SEED = 11


@pytest.fixture(scope="module")
def model():
    """(bfloat16 engine, 32-bit engine, plain weights) over one set of random weights."""
    import plain_random as R
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.weights import random_tensors_on_device
    cfg = u.config_from_dict(SIZES)
    spec = u.model_spec_for(cfg)
    specs = spec.weight_specs()
    t16 = random_tensors_on_device(specs, SEED, torch.bfloat16, "cuda:0")
    t32 = {k: v.float() for k, v in t16.items()}
    e16 = Engine(spec, t16, dtype="bfloat16", max_tokens=2048, max_seqs=4, max_step_tokens=512, poison_cache=True)
    e32 = Engine(spec, t32, dtype="float32", max_tokens=2048, max_seqs=4, max_step_tokens=512, poison_cache=True)
    # the oracle's weights: matrices as a bfloat16 folder would hold them, vectors in 32-bit, kept as
    # float32 arrays (exact), widened by numpy where they are used
    w = {s.name: R.tensor(SEED, s.name, s.shape, s.init, "bfloat16" if s.kind == "matrix" else "float32") for s in specs}
    # the device's draw is the host's, bit for bit, at these sizes too
    for name in ("model.layers.1.mlp.down_proj.weight", "model.layers.0.self_attn.k_norm.weight", "lm_head.weight"):
        assert np.array_equal(t16[name].float().cpu().numpy().view(np.uint32), w[name].view(np.uint32)), name
    # the embedding rows and the norm weights start the float64 arithmetic; the large matrices stay
    # float32 in memory and numpy widens each where a product uses it
    for name in w:
        if w[name].ndim == 1 or name == "model.embed_tokens.weight":
            w[name] = w[name].astype(np.float64)
    return {"bfloat16": e16, "float32": e32}, w


_refs: dict = {}


def _ref(w, ids):
    import plain_qwen3 as P
    key = tuple(ids)
    if key not in _refs:
        _refs[key] = P.forward(SIZES, w, ids)
        assert _refs[key].dtype == np.float64
    return _refs[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_and_last_32_one_by_one_at_real_widths(model, dtype):
    engines, w = model
    eng = engines[dtype]
    rng = np.random.default_rng(3)
    ids = rng.integers(0, SIZES["vocab_size"], size=150).tolist()
    ref = _ref(w, ids)
    assert np.abs(ref).max() > 1.0                               # logits with range, not a flat vector
    s = eng.open(1)
    whole = eng.step(s, [ids], [list(range(150))]).cpu().numpy()
    eng.close(s)
    err, bound = close_enough(whole, ref, dtype, 2)
    assert err <= bound, f"whole [{dtype}]: {err:.3e} > {bound:.3e}"
    s = eng.open(1)
    rows = [eng.step(s, [ids[:118]], [list(range(118))]).cpu().numpy()]
    for t in range(118, 150):
        rows.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    got = np.concatenate(rows)
    err, bound = close_enough(got, ref, dtype, 2)
    if err > bound:
        bad = int(np.argmax(np.abs(got - ref).max(axis=1) > bound))
        pytest.fail(f"last 32 one by one [{dtype}]: {err:.3e} > {bound:.3e}, first bad position {bad}")
    eng.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_at_real_widths(model, dtype):
    engines, w = model
    eng = engines[dtype]
    rng = np.random.default_rng(4)
    plens, dlens = [3, 70, 130, 17], [6, 2, 4, 6]
    seqs = [rng.integers(0, SIZES["vocab_size"], size=p + d).tolist() for p, d in zip(plens, dlens)]
    for round_ in range(2):                                      # the second round uses the slots again
        slots = eng.open(4)
        out = eng.step(slots, [s[:p] for s, p in zip(seqs, plens)], [list(range(p)) for p in plens]).cpu().numpy()
        got, o = [], 0
        for p in plens:
            got.append([out[o:o + p]])
            o += p
        live = [0, 1, 2, 3]
        for t in range(max(dlens)):
            for i in [i for i in live if t >= dlens[i]]:
                eng.close([slots[i]])
                live.remove(i)
            out = eng.step([slots[i] for i in live], [[seqs[i][plens[i] + t]] for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
        eng.close([slots[i] for i in live])
        assert eng.cache.pages_held() == 0
        for i, ids in enumerate(seqs):
            g = np.concatenate(got[i])
            err, bound = close_enough(g, _ref(w, ids), dtype, 2)
            assert err <= bound, f"round {round_} request {i} [{dtype}]: {err:.3e} > {bound:.3e}"
    eng.check_errors()
