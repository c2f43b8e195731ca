"""The generation loop's decisions with a fake engine and a fake sampler (no GPU): batches,
stop tokens, sequences that end earlier, slots given back, nothing fed after the end."""
import pytest

from ultima_b200.engine.generate import generate, plan_batches
from ultima_b200.sampling import SamplingParams


class FakeEngine:
    """Logits are stand-ins: row i is (slot, position, last token) of the sequence it belongs to."""

    def __init__(self, n_slots=4, max_tokens=4096, max_context=64):
        self.free = list(range(n_slots))[::-1]
        self.len = {}
        self.max_tokens, self.max_context = max_tokens, max_context
        self.calls, self.closed, self.max_live = [], [], 0

    def open(self, n):
        assert n <= len(self.free), "more sequences than slots"
        got = [self.free.pop() for _ in range(n)]
        for s in got:
            self.len[s] = 0
        self.max_live = max(self.max_live, len(self.len))
        return got

    def close(self, slots):
        for s in slots:
            assert s in self.len, "slot freed twice"
            del self.len[s]
            self.free.append(s)
            self.closed.append(s)

    def step(self, slots, tokens, want):
        assert want is None
        rows = []
        for s, t in zip(slots, tokens):
            assert s in self.len and len(t) >= 1
            self.len[s] += len(t)
            rows.append((s, self.len[s], t[-1]))
        self.calls.append([(s, list(t)) for s, t in zip(slots, tokens)])
        return rows


def scripted(script):
    """A sampler that gives request r (recognised by its prompt's last token at counter 0, then by
    the token fed) the tokens of script[r] one after another."""
    state = {}

    def sample(rows, params, streams, counters, recents):
        out = []
        for (slot, pos, last), stream, c in zip(rows, streams, counters):
            out.append(script[stream][c])
        return out
    return sample


def test_plan_batches_by_count_and_by_tokens():
    assert plan_batches([5, 5, 5, 5, 5], 2, 10_000, [3] * 5) == [[0, 1], [2, 3], [4]]
    # 60 + 10 -> 128 positions each (rounded up to pages of 64): two fit into 256
    assert plan_batches([60, 60, 60], 8, 256, [10] * 3) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="cache holds"):
        plan_batches([300], 8, 256, [10])


def _run(engine, script, prompts, n_predict, stop=(), max_batch=4):
    # streams are replaced by request indices so the scripted sampler can find its script
    import ultima_b200.engine.generate as G
    orig = G.stream_seed
    G.stream_seed = lambda seed, i: i
    try:
        return generate(engine, scripted(script), prompts, SamplingParams(), n_predict, stop,
                        max_batch=max_batch)
    finally:
        G.stream_seed = orig


def test_stop_token_is_neither_emitted_nor_fed_and_slot_comes_back_early():
    eng = FakeEngine()
    script = {0: [7, 8, 99, 1], 1: [5, 6, 7, 8, 9, 10]}
    out = _run(eng, script, [[1, 2, 3], [4]], 6, stop=(99,))
    assert out[0].tokens == [7, 8] and out[0].finish_reason == "stop"
    assert out[1].tokens == [5, 6, 7, 8, 9, 10] and out[1].finish_reason == "length"
    fed = [t for call in eng.calls[1:] for (_, t) in call]
    assert [99] not in fed                       # the stop token is never fed
    assert [10] not in fed                       # nor is the last sampled token
    # after request 0 stopped, steps carry one sequence only
    assert [len(c) for c in eng.calls] == [2, 2, 2, 1, 1, 1]
    assert sorted(eng.closed) == [0, 1] and eng.closed[0] == 0 and not eng.len


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(n_slots=2)
    script = {i: [i + 10] * 3 for i in range(5)}
    out = _run(eng, script, [[i + 1] * (i + 1) for i in range(5)], 3, max_batch=2)
    assert [g.tokens for g in out] == [[i + 10] * 3 for i in range(5)]
    assert eng.max_live == 2 and len(eng.closed) == 5 and not eng.len
    # each batch begins with its prompts, of unequal lengths, in one step
    firsts = [c for c in eng.calls if any(len(t) > 1 for _, t in c) or c[0][1] == [1]]
    assert [[len(t) for _, t in c] for c in firsts] == [[1, 2], [3, 4], [5]]


def test_per_request_lengths_and_zero_new_tokens():
    eng = FakeEngine()
    script = {0: [1, 2, 3], 1: [4, 5, 6], 2: [7, 8, 9]}
    out = _run(eng, script, [[1], [2], [3]], [1, 0, 3])
    assert [g.tokens for g in out] == [[1], [], [7, 8, 9]]
    assert [len(c) for c in eng.calls] == [2, 1, 1] and not eng.len


def test_context_overflow_is_refused_before_anything_runs():
    eng = FakeEngine(max_context=8)
    with pytest.raises(ValueError, match="does not fit the context"):
        _run(eng, {0: [1] * 9}, [[1, 2, 3]], 6)
    assert not eng.calls and not eng.len
    with pytest.raises(ValueError, match="empty prompt"):
        _run(eng, {0: [1]}, [[]], 1)


def test_slots_are_given_back_when_a_step_fails():
    class Boom(FakeEngine):
        def step(self, slots, tokens, want):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step(slots, tokens, want)
    eng = Boom()
    with pytest.raises(RuntimeError, match="boom"):
        _run(eng, {0: [1, 2, 3], 1: [1, 2, 3]}, [[1], [2]], 3)
    assert not eng.len and len(eng.free) == 4


def test_sampling_params_defaults_follow_the_reference():
    p = SamplingParams()
    assert p.greedy and not p.uses_history and p.top_k == 0 and p.top_p == 1.0
    s = SamplingParams.server_defaults()
    assert (s.temperature, s.top_k, s.top_p, s.min_p, s.rep_penalty, s.repeat_last_n) == (0.2, 40, 0.95, 0.05, 1.1, 64)
    assert (s.dry_multiplier, s.dry_base, s.dry_allowed_len, s.dry_last_n) == (0.8, 1.75, 2, 512)
    assert s.history_window() == 512
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1).validate()


def test_penalties_look_back_on_the_prompt_and_then_on_what_was_generated():
    """The reference pushes the prompt into its sampler's window before the first draw
    (apps/ultima-cli/main.cpp:664, src/server/http_server.cpp:163)."""
    import ultima_b200.engine.generate as G
    eng = FakeEngine()
    seen_by_sampler = []

    def sample(rows, params, streams, counters, recents):
        seen_by_sampler.append([list(r) for r in recents])
        return [50 + c for c in counters]
    with_history = SamplingParams(rep_penalty=1.3, repeat_last_n=8)
    plain = SamplingParams()
    generate(eng, sample, [[1, 2, 3], [4]], [with_history, plain], 3, ())
    assert [s[0] for s in seen_by_sampler] == [[1, 2, 3], [1, 2, 3, 50], [1, 2, 3, 50, 51]]
    assert all(s[1] == [] for s in seen_by_sampler)          # no history kept where nothing reads it
