"""The Tiny B workload end to end: four prompts of 1, 7, 30 and 64 tokens, 16 tokens each drawn at
temperature 0.8 from a fixed seed through the entry point, in 32-bit.  Every drawn token is checked
against the host's rule applied to the plain implementation's logits of the sequence so far: the
ladder of src/sampler/sampler.cpp:230-277 (here only the temperature), the inverse CDF, and the
uniform number of (seed, request, tokens drawn so far).  The engine's 32-bit logits are within 2e-5 of
the plain ones (the bound of the model tests), so its CDF is within 2.5e-5 of the plain CDF at this
temperature; a draw whose uniform number lies that close to a step of the plain CDF may fall either
way and is not compared (a few of the 64)."""
import numpy as np
import pytest


pytestmark = pytest.mark.gpu


def test_tiny_b_sampled_ids_follow_the_host_rule_on_plain_logits(model_dirs, plain_models):
    import plain_qwen3 as P
    import ultima_b200 as u
    from test_sampling_gpu import host_ladder
    from ultima_b200.sampling import SamplingParams, uniform_of
    from ultima_b200.sampling.sampler import stream_seed
    name, seed, n_new = "B", 1234, 16
    cfg, w = plain_models(name, "float32")
    V = cfg["vocab_size"]
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, V, size=n).tolist() for n in (1, 7, 30, 64)]
    llm = u.LLM(model_dirs(name, "float32"), dtype="float32", n_ctx=128, max_batch=4)
    params = SamplingParams(temperature=0.8)
    outs = llm.generate(prompts, n_predict=n_new, temp=0.8, seed=seed, stop_token_ids=())
    assert [len(o.tokens) for o in outs] == [n_new] * 4
    compared = 0
    for i, (prompt, out) in enumerate(zip(prompts, outs)):
        stream = stream_seed(seed, i)
        for t in range(n_new):
            logits = P.forward(cfg, w, prompt + out.tokens[:t])[-1]
            probs, _ = host_ladder(logits, params, [])
            cdf = np.cumsum(probs)
            x = uniform_of(stream, t)
            if np.abs(cdf - x).min() < 2.5e-5:
                continue
            want = int(np.searchsorted(cdf, x, side="right"))
            assert out.tokens[t] == want, (i, t, out.tokens[t], want, x)
            compared += 1
    assert compared >= 52
    # each request alone draws the same tokens: a sequence's stream does not depend on its batch
    alone = u.LLM(model_dirs(name, "float32"), dtype="float32", n_ctx=128, max_batch=1)
    solo = alone.generate(prompts, n_predict=n_new, temp=0.8, seed=seed, stop_token_ids=())
    assert [o.tokens for o in solo] == [o.tokens for o in outs]
    # and the device kept time of its own steps
    st = llm.last_stats
    assert st.device_prefill_ms > 0 and len(st.device_step_ms) == n_new - 1 and min(st.device_step_ms) > 0
