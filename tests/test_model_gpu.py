"""The engine against the plain implementation on the GPU, in 32-bit and in bfloat16:
requests alone and whole; the last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again; long
decoding; the first tokens of a sequence."""
import numpy as np
import pytest
import torch

from conftest import TINY, random_ids, close_enough

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C"]


def _engine(model_dirs, name, dtype, **kw):
    from ultima_b200.engine import Engine
    kw.setdefault("max_tokens", 2048)
    kw.setdefault("poison_cache", True)
    return Engine.from_dir(model_dirs(name, "bfloat16"), dtype=dtype, **kw)


def _plain_logits(plain_models, name, ids):
    import plain_qwen3 as P
    cfg, w = plain_models(name, "bfloat16")
    return P.forward(cfg, w, ids)


def _check(got, ref, dtype, name, what):
    err, bound = close_enough(got, ref, dtype, TINY[name]["num_hidden_layers"])
    assert err <= bound, f"{what} [{name} {dtype}]: max |logit error| {err:.3e} > {bound:.3e}"
    return err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_request_alone(model_dirs, plain_models, name, dtype):
    eng = _engine(model_dirs, name, dtype)
    V = TINY[name]["vocab_size"]
    for seed, n in ((1, 1), (2, 5), (3, 64), (4, 97)):
        ids = random_ids(seed, n, V)
        s = eng.open(1)
        got = eng.step(s, [ids], [list(range(n))]).cpu().numpy()
        eng.close(s)
        _check(got, _plain_logits(plain_models, name, ids), dtype, name, f"whole, {n} tokens")
    assert eng.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_one_by_one(model_dirs, plain_models, name, dtype):
    eng = _engine(model_dirs, name, dtype)
    V = TINY[name]["vocab_size"]
    for seed, n in ((5, 20), (6, 33), (7, 100)):
        ids = random_ids(seed, n, V)
        ref = _plain_logits(plain_models, name, ids)
        head = max(0, n - 32)
        s = eng.open(1)
        rows = []
        if head:
            rows.append(eng.step(s, [ids[:head]], [list(range(head))]).cpu().numpy())
        for t in range(head, n):
            rows.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
        eng.close(s)
        got = np.concatenate(rows, axis=0)
        err, bound = close_enough(got, ref, dtype, TINY[name]["num_hidden_layers"])
        if err > bound:
            bad = int(np.argmax(np.abs(got - ref).max(axis=1)))
            pytest.fail(f"last-32 [{name} {dtype}] n={n}: error {err:.3e} > {bound:.3e}; first bad "
                        f"position {bad} (prompt part ends at {head})")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_slots_reused(model_dirs, plain_models, name, dtype):
    """Three batches one after another in a cache that only just holds one of them."""
    V = TINY[name]["vocab_size"]
    lens = [[5, 11, 17, 40], [1, 7, 30, 64], [33, 2, 65, 9]]
    decode = [[3, 9, 1, 6], [8, 2, 5, 0], [4, 7, 0, 10]]
    eng = _engine(model_dirs, name, dtype, max_tokens=4 * 128, max_seqs=4)
    for b, (pl, dl) in enumerate(zip(lens, decode)):
        full = [random_ids(100 + 10 * b + i, p + d, V) for i, (p, d) in enumerate(zip(pl, dl))]
        refs = [_plain_logits(plain_models, name, ids) for ids in full]
        slots = eng.open(len(full))
        got = [[] for _ in full]
        out = eng.step(slots, [ids[:p] for ids, p in zip(full, pl)],
                       [list(range(p)) for p in pl]).cpu().numpy()
        o = 0
        for i, p in enumerate(pl):
            got[i].append(out[o:o + p])
            o += p
        live = list(range(len(full)))
        for t in range(max(dl)):
            for i in [i for i in live if dl[i] <= t]:      # shorter requests end earlier
                eng.close([slots[i]])
                live.remove(i)
            if not live:
                break
            out = eng.step([slots[i] for i in live], [[full[i][pl[i] + t]] for i in live],
                           [[0]] * len(live)).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
        eng.close([slots[i] for i in live])
        assert eng.cache.pages_held() == 0 and eng.cache.slots.n_free == 4
        for i, ref in enumerate(refs):
            g = np.concatenate(got[i], axis=0)
            err, bound = close_enough(g, ref, dtype, TINY[name]["num_hidden_layers"])
            if err > bound:
                bad = int(np.argmax(np.abs(g - ref).max(axis=1)))
                pytest.fail(f"batch {b} request {i} [{name} {dtype}]: error {err:.3e} > {bound:.3e} "
                            f"first at position {bad} (prompt {pl[i]}, decoded {dl[i]})")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(model_dirs, plain_models, name, dtype):
    """A short prompt, then token by token across several pages (and past the window)."""
    V = TINY[name]["vocab_size"]
    n = min(TINY[name]["max_position_embeddings"], 200)
    ids = random_ids(42, n, V)
    ref = _plain_logits(plain_models, name, ids)
    eng = _engine(model_dirs, name, dtype)
    s = eng.open(1)
    rows = [eng.step(s, [ids[:3]], [[0, 1, 2]]).cpu().numpy()]
    for t in range(3, n):
        rows.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    got = np.concatenate(rows, axis=0)
    err, bound = close_enough(got, ref, dtype, TINY[name]["num_hidden_layers"])
    if err > bound:
        bad = int(np.argmax(np.abs(got - ref).max(axis=1) > bound))
        pytest.fail(f"long decode [{name} {dtype}]: error {err:.3e} > {bound:.3e}, first bad position {bad}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_decoding_around_a_window_ring_of_one_page(model_dirs, plain_models, name, dtype):
    """Passes of at most 16 tokens make the windowed layers' ring as small as it can be: one page of 64
    positions for windows of 20 (C, head size 48) and 40 (D, head size 64).  A prompt of 50 tokens in four
    passes, then token by token to 200 positions: the ring wraps three times, every page of it is used
    again and again, and the page of the new position always holds the window's oldest keys too."""
    from ultima_b200.cache import PAGE
    V = TINY[name]["vocab_size"]
    n = 200
    ids = random_ids(77, n, V)
    ref = _plain_logits(plain_models, name, ids)
    eng = _engine(model_dirs, name, dtype, max_step_tokens=16)
    rings = sorted(g.ring for g in eng.cache.kv_groups)
    assert rings[0] == PAGE and rings[-1] > PAGE             # the windowed group wraps, the full one does not
    s = eng.open(1)
    rows = [eng.step(s, [ids[:50]], [list(range(50))]).cpu().numpy()]
    for t in range(50, n):
        rows.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    eng.check_errors()
    got = np.concatenate(rows, axis=0)
    err, bound = close_enough(got, ref, dtype, TINY[name]["num_hidden_layers"])
    if err > bound:
        bad = int(np.argmax(np.abs(got - ref).max(axis=1) > bound))
        pytest.fail(f"window ring [{name} {dtype}]: error {err:.3e} > {bound:.3e}, first bad position {bad}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_want_subsets(model_dirs, plain_models, dtype):
    """Position 0 alone, a prompt of one token, and wanted places given out of order."""
    name = "B"
    V = TINY[name]["vocab_size"]
    eng = _engine(model_dirs, name, dtype)
    a, b = random_ids(1, 1, V), random_ids(2, 9, V)
    sl = eng.open(2)
    out = eng.step(sl, [a, b], [[0], [8, 0, 3]]).cpu().numpy()
    eng.close(sl)
    ra, rb = _plain_logits(plain_models, name, a), _plain_logits(plain_models, name, b)
    _check(out[0:1], ra, dtype, name, "single-token prompt")
    _check(out[1:4], rb[[8, 0, 3]], dtype, name, "wanted places out of order")
    # nothing wanted: the step still fills the cache
    sl = eng.open(1)
    assert eng.step(sl, [b[:4]], [[]]).shape[0] == 0
    got = eng.step(sl, [b[4:]], [[4]]).cpu().numpy()
    eng.close(sl)
    _check(got, rb[8:9], dtype, name, "continuation after a step with nothing wanted")


@pytest.mark.parametrize("dtype", DTYPES)
def test_passes_inside_a_step_change_nothing(model_dirs, plain_models, dtype):
    """A step cut into several passes (small max_step_tokens) gives the same logits."""
    name = "C"
    V = TINY[name]["vocab_size"]
    ids = [random_ids(50 + i, n, V) for i, n in enumerate((70, 13, 41))]
    eng = _engine(model_dirs, name, dtype, max_step_tokens=32)
    sl = eng.open(3)
    out = eng.step(sl, ids, [list(range(len(t))) for t in ids]).cpu().numpy()
    eng.close(sl)
    o = 0
    for t in ids:
        _check(out[o:o + len(t)], _plain_logits(plain_models, name, t), dtype, name, "passes")
        o += len(t)


def test_weights_stored_in_32_bit_stay_32_bit_on_the_bfloat16_path(model_dirs, plain_models):
    """A folder whose tensors are float32, run with dtype bfloat16: the weights are not rounded (their
    products run on the CUDA-core kernel), activations and cache are bfloat16."""
    import plain_qwen3 as P
    import torch
    from ultima_b200.engine import Engine
    name = "B"
    eng = Engine.from_dir(model_dirs(name, "float32"), dtype="bfloat16", max_tokens=1024, poison_cache=True)
    att = eng.model.layers[0].mixer
    assert att.wqkv.dtype == torch.float32 and eng.model.head.weight.dtype == torch.float32
    assert eng.cache.kv_groups[0].k.dtype == torch.bfloat16
    cfg, w = plain_models(name, "float32")
    ids = random_ids(77, 50, TINY[name]["vocab_size"])
    s = eng.open(1)
    rows = [eng.step(s, [ids[:40]], [list(range(40))]).cpu().numpy()]
    for t in range(40, 50):
        rows.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    _check(np.concatenate(rows), P.forward(cfg, w, ids), "bfloat16", name, "float32 weights on the bfloat16 path")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_fit_no_tensor_core_kernel(model_dirs, plain_models, dtype):
    """Rows of 100 values, 5 heads of size 24, an inner size of 131, a vocabulary of 257: on the
    bfloat16 path every product goes to the CUDA-core kernel and attention to the float32-accumulating
    kernel, and the logits are still the plain implementation's: whole, and the end one by one."""
    eng = _engine(model_dirs, "F", dtype)
    ids = random_ids(31, 90, 257)
    ref = _plain_logits(plain_models, "F", ids)
    s = eng.open(1)
    got = eng.step(s, [ids], [list(range(90))]).cpu().numpy()
    eng.close(s)
    _check(got, ref, dtype, "F", "whole, 90 tokens")
    s = eng.open(2)
    rows = [eng.step(s, [ids[:70], ids[:5]], [list(range(70)), []]).cpu().numpy()]
    for t in range(70, 90):
        rows.append(eng.step([s[0]], [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    _check(np.concatenate(rows), ref, dtype, "F", "70 tokens, then one by one beside a second sequence")
    eng.check_errors()
    assert eng.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "E"])
def test_logits_with_range(tmp_path, name, dtype):
    """The same comparisons on a model whose matrices are five times as large as a random model's, so
    that its logits reach well beyond 1: the bound, which is relative to the largest logit, is then
    small beside the logits' spread and a key weighted wrongly would show, not only a key lost."""
    import json
    import os
    import plain_qwen3 as P
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.weights import random_tensors, write_safetensors
    cfg = u.config_from_dict(TINY[name])
    spec = u.model_spec_for(cfg)
    tensors = random_tensors(spec.weight_specs(), 13, torch.bfloat16)
    for s_ in spec.weight_specs():
        if s_.kind == "matrix":
            tensors[s_.name] = (tensors[s_.name].float() * 5.0).to(torch.bfloat16)
    d = str(tmp_path / "wide")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    pc, pw = P.read_folder(d)
    V, L = cfg.vocab_size, cfg.num_hidden_layers
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=1024, max_seqs=3, poison_cache=True)
    seqs = [random_ids(200 + i, n, V) for i, n in enumerate((100, 37, 66))]
    refs = [P.forward(pc, pw, s_) for s_ in seqs]
    assert min(float(np.abs(r).max()) for r in refs) > 3.0 and min(float(r.std()) for r in refs) > 0.5
    # whole; then prompts together and the last 32 tokens one by one, the shorter ones leaving first
    sl = eng.open(1)
    got = eng.step(sl, [seqs[0]], [list(range(100))]).cpu().numpy()
    eng.close(sl)
    err, bound = close_enough(got, refs[0], dtype, L)
    assert err <= bound, f"whole [{name} {dtype}]: {err:.3e} > {bound:.3e} (spread {refs[0].std():.2f})"
    cut = [len(s_) - 32 for s_ in seqs]
    sl = eng.open(3)
    out = eng.step(sl, [s_[:c] for s_, c in zip(seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
    rows, o = [], 0
    for c in cut:
        rows.append([out[o:o + c]])
        o += c
    for t in range(32):
        out = eng.step(sl, [[s_[c + t]] for s_, c in zip(seqs, cut)]).cpu().numpy()
        for i in range(3):
            rows[i].append(out[i:i + 1])
    eng.close(sl)
    for i in range(3):
        g = np.concatenate(rows[i])
        err, bound = close_enough(g, refs[i], dtype, L)
        assert err <= bound, f"request {i} [{name} {dtype}]: {err:.3e} > {bound:.3e} (spread {refs[i].std():.2f})"
