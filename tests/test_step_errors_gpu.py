"""Every refusal of the step function: the error is raised on the host, nothing is launched and the
cache is as it was.  Then the device-side flag (a token id that only the device sees), and prefix
reuse: a slot cut back to a shared prefix and continued, against the plain implementation.
The reference refuses a token id outside the vocabulary (src/model/qwen_model.cpp:147-152) and a
prompt that does not fit the context (apps/ultima-cli/main.cpp:637-641), and truncates a slot to the
common prefix of its tokens and a new prompt (src/kv_cache/kv_cache.cpp:141-157)."""
import numpy as np
import pytest
import torch

from conftest import TINY, close_enough, random_ids

pytestmark = pytest.mark.gpu


def _engine(model_dirs, name="A", dtype="float32", **kw):
    from ultima_b200.engine import Engine
    kw.setdefault("max_tokens", 512)
    return Engine.from_dir(model_dirs(name, "bfloat16"), dtype=dtype, **kw)


def _refused(eng, match, fn):
    """``fn`` raises a StepError that says ``match``; no kernel was launched, no length or page moved."""
    from ultima_b200.engine import StepError
    before = (eng.rt.launches, list(eng.cache.slots.length), eng.cache.pages_held(), eng.cache.slots.n_free)
    with pytest.raises(StepError, match=match):
        fn()
    assert (eng.rt.launches, list(eng.cache.slots.length), eng.cache.pages_held(), eng.cache.slots.n_free) == before


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_refusal_of_a_step(model_dirs, dtype):
    eng = _engine(model_dirs, "A", dtype, max_tokens=256, max_seqs=3, max_context=100)
    V = TINY["A"]["vocab_size"]
    a, b = eng.open(2)
    eng.step([a, b], [[1, 2, 3], [4]], None)                     # a is at 3 positions, b at 1
    free = [s for s in range(3) if s not in (a, b)][0]
    # ---- the general step
    _refused(eng, "one token list for each slot", lambda: eng.step([a, b], [[1, 2]], None))
    _refused(eng, "one list of wanted places for each slot", lambda: eng.step([a, b], [[1, 2], [3]], [[0]]))
    _refused(eng, "named twice", lambda: eng.step([a, a], [[1, 2], [3, 4]], None))
    _refused(eng, "is not held", lambda: eng.step([a, free], [[1, 2], [3, 4]], None))
    _refused(eng, "does not exist", lambda: eng.step([a, 17], [[1, 2], [3, 4]], None))
    _refused(eng, "brings no token", lambda: eng.step([a, b], [[1, 2], []], [[0], [0]]))
    _refused(eng, "flat lists of integers", lambda: eng.step([a], [[[1, 2], [3, 4]]], [[0]]))
    _refused(eng, "flat lists of integers", lambda: eng.step([a], [[0.5, 2.0]], [[0]]))
    _refused(eng, f"token id {V} is outside the vocabulary", lambda: eng.step([a, b], [[1, V], [3, 4]], None))
    _refused(eng, "token id -1 is outside the vocabulary", lambda: eng.step([a, b], [[1, 2], [-1, 4]], None))
    _refused(eng, "wanted place 2 is outside the 2 tokens", lambda: eng.step([a, b], [[1, 2], [3, 4]], [[0], [2]]))
    _refused(eng, "wanted place -1 is outside", lambda: eng.step([a, b], [[1, 2], [3, 4]], [[-1], [0]]))
    _refused(eng, "would reach 101 positions; the limit is 100", lambda: eng.step([a], [[5] * 98], None))
    # ---- the common decode step (one token each, nothing said about wanted places)
    _refused(eng, "named twice", lambda: eng.step([b, b], [[1], [2]]))
    _refused(eng, "is not held", lambda: eng.step([free], [[1]]))
    _refused(eng, f"token id {V + 5} is outside the vocabulary", lambda: eng.step([a, b], [[1], [V + 5]]))
    # ---- the cache is full: 256 positions = 4 pages; a holds 1, b holds 1; c takes the other two
    c = eng.open(1)[0]
    eng.step([c], [[7] * 100], [[]])
    _refused(eng, "cache is full", lambda: eng.step([a], [[5] * 70], None))            # a would need a second page
    _refused(eng, "would reach 101 positions", lambda: eng.step([c], [[1]]))           # the context, in the decode step
    eng.step([a], [[5] * 61], [[]])                                                    # a at 64: the page's edge
    _refused(eng, "cache is full", lambda: eng.step([a, b], [[1], [2]]))               # one token more needs a page
    # after all that the engine still steps
    out = eng.step([b], [[9]])
    assert out.shape == (1, V) and torch.isfinite(out).all()
    eng.check_errors()
    eng.close([a, b, c])
    assert eng.cache.pages_held() == 0 and eng.cache.slots.n_free == 3


def test_refusals_of_steps_fed_from_the_device(model_dirs):
    from ultima_b200.engine import StepError
    eng = _engine(model_dirs, "A", "float32", max_seqs=2, max_context=70)     # 32-bit: sums in a fixed order, so equal bits
    V = TINY["A"]["vocab_size"]
    a, b = eng.open(2)
    eng.step([a, b], [[1, 2, 3], [4]], None)
    good = torch.tensor([5, 6], dtype=torch.int32, device=eng.device)
    _refused(eng, "named twice", lambda: eng.step_fed([a, a], good))
    _refused(eng, "int32 on the engine's device", lambda: eng.step_fed([a, b], good.long()))
    _refused(eng, "int32 on the engine's device", lambda: eng.step_fed([a, b], good.cpu()))
    _refused(eng, "int32 on the engine's device", lambda: eng.step_fed([a, b], good[:1]))
    plain = _engine(model_dirs, "A", "float32", use_graphs=False)
    s = plain.open(1)
    with pytest.raises(StepError, match="does not replay captured decode steps"):
        plain.step_fed(s, good)
    # the same logits as the step that takes its ids from the host
    want = eng.step([a, b], [[5], [6]]).clone()
    eng.truncate(a, 3), eng.truncate(b, 1)
    got = eng.step_fed([a, b], good)
    assert torch.equal(got, want)
    # an id that only the device sees: the embedding kernel raises the flag, check_errors reports it
    eng.check_errors()
    bad = torch.tensor([5, V + 3], dtype=torch.int32, device=eng.device)
    eng.step_fed([a, b], bad)
    with pytest.raises(RuntimeError, match="outside the vocabulary"):
        eng.check_errors()
    eng.check_errors()                                                # the flag is cleared by the report
    # a step that would pass the context is refused here too
    eng.step([a], [[1] * 65], [[]])                                   # a holds 70 positions: the limit
    _refused(eng, "would reach 71 positions", lambda: eng.step_fed([a, b], good))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_truncate_to_a_shared_prefix_and_continue(model_dirs, plain_models, dtype):
    """Two prompts that share their first 70 tokens, one slot: run the first, cut the slot back to the
    shared prefix (a page and six positions), continue with the second's tail, then decode.  Every
    logit after the cut is the plain implementation's for the second prompt."""
    import plain_qwen3 as P
    from ultima_b200.cache import CacheError
    name = "A"
    cfg, w = plain_models(name, "bfloat16")
    V = cfg["vocab_size"]
    eng = _engine(model_dirs, name, dtype, max_tokens=256, max_seqs=1, poison_cache=True)
    shared = random_ids(1, 70, V)
    first = shared + random_ids(2, 40, V)
    second = shared + random_ids(3, 30, V)
    ref = P.forward(cfg, w, second)
    s = eng.open(1)
    eng.step(s, [first], [[len(first) - 1]])
    assert eng.length(s[0]) == 110 and eng.cache.pages_held() == 2
    eng.truncate(s[0], 70)
    assert eng.length(s[0]) == 70 and eng.cache.pages_held() == 2
    rows = [eng.step(s, [second[70:90]], [list(range(20))]).cpu().numpy()]
    for t in range(90, 100):
        rows.append(eng.step(s, [[second[t]]], [[0]]).cpu().numpy())
    got = np.concatenate(rows)
    err, bound = close_enough(got, ref[70:100], dtype, cfg["num_hidden_layers"])
    assert err <= bound, (err, bound)
    # back to a page's edge frees the page behind it; to zero frees all
    eng.truncate(s[0], 64)
    assert eng.cache.pages_held() == 1
    got = eng.step(s, [second[64:72]], [[7]]).cpu().numpy()
    err, bound = close_enough(got, ref[71:72], dtype, cfg["num_hidden_layers"])
    assert err <= bound
    with pytest.raises(CacheError, match="cannot truncate"):
        eng.truncate(s[0], 500)
    eng.truncate(s[0], 0)
    assert eng.cache.pages_held() == 0 and eng.length(s[0]) == 0
    got = eng.step(s, [second[:5]], [[4]]).cpu().numpy()
    err, bound = close_enough(got, ref[4:5], dtype, cfg["num_hidden_layers"])
    assert err <= bound
    eng.close(s)


def test_truncate_is_refused_where_a_window_has_let_go_of_the_past(model_dirs):
    from ultima_b200.cache import CacheError
    eng = _engine(model_dirs, "C", "float32")                      # layers with a window of 20
    s = eng.open(1)
    eng.step(s, [random_ids(4, 60, TINY["C"]["vocab_size"])], None)
    with pytest.raises(CacheError, match="only be truncated to its start"):
        eng.truncate(s[0], 30)
    eng.truncate(s[0], 0)                                          # to the start it can
    assert eng.length(s[0]) == 0
    eng.close(s)


def test_a_head_size_no_kernel_takes_is_refused_when_the_engine_is_built():
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.weights import random_tensors
    cfg = u.config_from_dict(dict(TINY["A"], head_dim=272, num_attention_heads=2, num_key_value_heads=1))
    spec = u.model_spec_for(cfg)
    tensors = {k: v.to("cuda:0") for k, v in random_tensors(spec.weight_specs(), 1).items()}
    for dtype in ("float32", "bfloat16"):
        with pytest.raises(ValueError, match="head size 272 is not one the kernels take"):
            Engine(spec, tensors, dtype=dtype, max_tokens=256)
