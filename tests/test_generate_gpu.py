"""Generation through the entry point against the plain implementation."""
import pytest

from conftest import random_ids

pytestmark = pytest.mark.gpu


def _flat_enough(cfg, w, ids, got):
    """Random weights give nearly flat logits; a greedy token is right when its plain logit is
    within float32 rounding of the plain maximum."""
    import plain_qwen3 as P
    lg = P.forward(cfg, w, ids)[-1]
    return lg.max() - lg[got] <= 1e-5


def test_greedy_three_prompts_match_the_plain_implementation(model_dirs, plain_models):
    """Tiny A: a batch of prompts of 5, 11 and 17 tokens, then 8 greedy tokens each, 32-bit."""
    import plain_qwen3 as P
    from ultima_b200 import LLM
    cfg, w = plain_models("A", "float32")
    llm = LLM(model_dirs("A", "float32"), dtype="float32", n_ctx=128, max_batch=4)
    prompts = [random_ids(i, n, 512) for i, n in enumerate((5, 11, 17))]
    outs = llm.generate(prompts, n_predict=8, temp=0.0)
    for p, g in zip(prompts, outs):
        assert len(g.tokens) == 8 and g.finish_reason == "length"
        ids = list(p)
        for t in g.tokens:
            assert _flat_enough(cfg, w, ids, t), "greedy token is not the plain maximum"
            ids.append(t)
    st = llm.last_stats
    assert st.prompt_tokens == 33 and st.generated_tokens == 24
    assert llm.engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_tokens_do_not_depend_on_the_batch(model_dirs, dtype):
    """Tiny B: prompts of 1, 7, 30 and 64 tokens, 16 tokens at temperature 0.8 from a fixed seed;
    each request alone gives the tokens it gives in the batch; stop tokens cut a sequence."""
    from ultima_b200 import LLM, SamplingParams
    llm = LLM(model_dirs("B", "bfloat16"), dtype=dtype, n_ctx=256, max_batch=4)
    prompts = [random_ids(10 + i, n, 1000) for i, n in enumerate((1, 7, 30, 64))]
    sp = SamplingParams(temperature=0.8)
    together = llm.generate(prompts, n_predict=16, seed=123, sampling=sp)
    assert all(len(g.tokens) == 16 for g in together)
    again = llm.generate(prompts, n_predict=16, seed=123, sampling=sp)
    assert [g.tokens for g in again] == [g.tokens for g in together]
    other = llm.generate(prompts, n_predict=16, seed=124, sampling=sp)
    assert [g.tokens for g in other] != [g.tokens for g in together]
    if dtype == "float32":
        small = LLM(model_dirs("B", "bfloat16"), dtype=dtype, n_ctx=256, max_batch=1)
        one_by_one = small.generate(prompts, n_predict=16, seed=123, sampling=sp)
        assert [g.tokens for g in one_by_one] == [g.tokens for g in together]
    # a stop token: the sequence ends before it, the others go on
    stop = together[2].tokens[5]
    cut = llm.generate(prompts, n_predict=16, seed=123, sampling=sp, stop_token_ids=[stop])
    k = together[2].tokens.index(stop)
    assert cut[2].tokens == together[2].tokens[:k] and cut[2].finish_reason == "stop"
    for i in (0, 1, 3):
        if stop not in together[i].tokens:
            assert cut[i].tokens == together[i].tokens
    assert llm.engine.cache.pages_held() == 0


def test_more_requests_than_slots_run_batch_after_batch(model_dirs, plain_models):
    from ultima_b200 import LLM
    cfg, w = plain_models("C", "bfloat16")
    llm = LLM(model_dirs("C", "bfloat16"), dtype="float32", n_ctx=128, max_batch=3)
    prompts = [random_ids(30 + i, 3 + 5 * i, 777) for i in range(7)]
    outs = llm.generate(prompts, n_predict=[2, 5, 1, 4, 3, 6, 2])
    assert [len(g.tokens) for g in outs] == [2, 5, 1, 4, 3, 6, 2]
    for p, g in zip(prompts, outs):
        ids = list(p)
        for t in g.tokens:
            assert _flat_enough(cfg, w, ids, t)
            ids.append(t)
    assert llm.engine.cache.slots.n_free == 3


def test_command_line_run(model_dirs, capsys):
    from ultima_b200.cli import main
    rc = main(["run", model_dirs("A", "float32"), "--prompt", "1,2,3;4,5", "--n-predict", "4",
               "--n-ctx", "64", "--dtype", "float32", "--show-tokens"])
    out = capsys.readouterr()
    assert rc == 0
    lines = [l for l in out.out.splitlines() if l and not l.startswith("prompt tokens")]
    assert len(lines) == 2 and all(len(l.split()) == 4 for l in lines)
    assert "gen tok" in out.err
    assert main(["run", model_dirs("A", "float32"), "--n-predict", "100", "--n-ctx", "64"]) == 1
    assert main(["run", model_dirs("A", "float32"), "--bogus"]) == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_queued_ahead_of_the_host_change_nothing(model_dirs, dtype):
    """With a sampler that hands its ids on without the host and an engine that takes them from the
    device, the loop queues the next step before it has seen this step's ids.  Tokens, finish reasons
    and what is left in the cache are those of the loop that waits for every step: with stop tokens
    that cut sequences at different steps, per-request lengths, seeded sampling and penalties."""
    from ultima_b200 import LLM
    from ultima_b200.engine.generate import generate
    from ultima_b200.sampling import SamplingParams
    llm = LLM(model_dirs("B", dtype), dtype=dtype, n_ctx=256, max_batch=8)
    assert llm.engine.feeds_from_device
    prompts = [random_ids(40 + i, n, 1000) for i, n in enumerate((1, 7, 30, 64, 3, 12))]
    cases = [(SamplingParams(), ()),
             (SamplingParams(temperature=0.9, top_k=50, rep_penalty=1.3, repeat_last_n=32), ()),
             (SamplingParams(temperature=1.2, top_p=0.95, frequency_penalty=0.3), None)]
    for sp, stop in cases:
        n_predict = [24, 9, 24, 17, 1, 24]
        waits = lambda *a: llm.sampler.sample(*a)          # a plain function: the loop cannot look ahead
        ref = generate(llm.engine, waits, prompts, sp, n_predict, stop or (), seed=5, max_batch=8)
        if stop is None:                                   # stop on tokens that really come up, early and late
            stop = (ref[0].tokens[5], ref[2].tokens[11], ref[5].tokens[20])
            ref = generate(llm.engine, waits, prompts, sp, n_predict, stop, seed=5, max_batch=8)
            assert any(g.finish_reason == "stop" for g in ref)
        got = generate(llm.engine, llm.sampler.sample, prompts, sp, n_predict, stop, seed=5, max_batch=8)
        assert [g.tokens for g in got] == [g.tokens for g in ref]
        assert [g.finish_reason for g in got] == [g.finish_reason for g in ref]
        assert llm.engine.cache.pages_held() == 0
        llm.engine.check_errors()
