"""The sampling kernel against a plain restatement of the same ladder on the host."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sampler(V):
    from ultima_b200.sampling import Sampler
    return Sampler(DEV, V)


def host_ladder(logits, p, recent):
    """The steps of src/sampler/sampler.cpp:230-277 on a float64 copy; returns the kept
    probabilities (zeros for masked entries), or the argmax for temperature <= 0."""
    x = np.array(logits, dtype=np.float64)
    V = len(x)
    for k, b in p.logit_bias.items():
        if 0 <= k < V:
            x[k] += b
    def counts(win):
        seg = recent[-win:] if win > 0 else []
        c = {}
        for t in seg:
            c[t] = c.get(t, 0) + 1
        return c, len(seg)
    if p.rep_penalty != 1.0 and p.repeat_last_n > 0:
        for t in counts(p.repeat_last_n)[0]:
            if 0 <= t < V:
                x[t] = x[t] / p.rep_penalty if x[t] > 0 else x[t] * p.rep_penalty
    if p.dry_multiplier > 0 and p.dry_last_n > 0:
        c, n = counts(p.dry_last_n)
        if n >= 2:
            for t, k in c.items():
                if k > p.dry_allowed_len and 0 <= t < V:
                    x[t] -= p.dry_multiplier * p.dry_base ** (k - p.dry_allowed_len)
    if p.frequency_penalty != 0 or p.presence_penalty != 0:
        for t, k in counts(max(p.repeat_last_n, p.dry_last_n))[0].items():
            if 0 <= t < V:
                x[t] -= k * p.frequency_penalty + p.presence_penalty
    if p.temperature <= 0:
        return int(np.argmax(x)), x
    x = x / p.temperature
    keep = np.ones(V, dtype=bool)
    if 0 < p.top_k < V:
        kth = np.sort(x)[-p.top_k]
        keep &= x >= kth
    def probs():
        e = np.where(keep, np.exp(x - x[keep].max()), 0.0)
        return e / e.sum()
    if 0 < p.top_p < 1:
        pr = probs()
        order = np.argsort(-pr, kind="stable")
        cum = np.cumsum(pr[order])
        cutoff = int(np.searchsorted(cum, p.top_p - 1e-12)) + 1
        thr = pr[order[cutoff - 1]]
        keep &= pr >= thr
    if p.min_p > 0:
        pr = probs()
        keep &= pr >= p.min_p * pr.max()
    return probs(), x


def test_greedy_takes_the_first_maximum():
    V = 1000
    s = _sampler(V)
    from ultima_b200.sampling import SamplingParams
    x = torch.zeros(3, V)
    x[0, [17, 400, 999]] = 2.0
    x[1, 999] = 1.0
    x[2] = -5.0
    got = s.sample(x.to(DEV), [SamplingParams()] * 3, [1, 2, 3], [0, 0, 0])
    assert got == [17, 999, 0]


def test_temperature_draw_follows_the_inverse_cdf_and_its_stream():
    from ultima_b200.sampling import SamplingParams, uniform_of
    from ultima_b200.sampling.sampler import stream_seed
    V = 777
    s = _sampler(V)
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(4, V, generator=g) * 2
    p = SamplingParams(temperature=0.8)
    streams = [stream_seed(11, i) for i in range(4)]
    for counter in range(6):
        got = s.sample(logits.to(DEV), [p] * 4, streams, [counter] * 4)
        for r in range(4):
            pr, _ = host_ladder(logits[r].numpy(), p, [])
            cdf = np.cumsum(pr)
            u = uniform_of(streams[r], counter)
            lo = cdf[got[r] - 1] if got[r] > 0 else 0.0
            assert lo - 1e-5 <= u <= cdf[got[r]] + 1e-5, (r, counter, got[r], u, lo, cdf[got[r]])
    # same stream and counter: same token, whatever the batch around it
    alone = s.sample(logits[2:3].to(DEV), [p], streams[2:3], [3])
    batch = s.sample(logits.to(DEV), [p] * 4, streams, [3] * 4)
    assert alone[0] == batch[2]
    # the draws follow the distribution: sharp logits, many counters
    sharp = torch.tensor([[0.0, math.log(3.0), -30.0, math.log(6.0)]]).repeat(2000, 1)
    ids = _sampler(4).sample(sharp.to(DEV), [SamplingParams(temperature=1.0)] * 2000, [5] * 2000, list(range(2000)))
    freq = np.bincount(ids, minlength=4) / 2000.0
    assert np.allclose(freq, [0.1, 0.3, 0.0, 0.6], atol=0.04)


@pytest.mark.parametrize("case", ["top_k", "top_p", "min_p", "all"])
def test_cuts_keep_the_same_set_as_the_host(case):
    from ultima_b200.sampling import SamplingParams
    V = 5003
    s = _sampler(V)
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(1, V, generator=g) * 3
    p = {"top_k": SamplingParams(temperature=0.7, top_k=12),
         "top_p": SamplingParams(temperature=1.3, top_p=0.6),
         "min_p": SamplingParams(temperature=1.0, min_p=0.2),
         "all": SamplingParams(temperature=0.9, top_k=40, top_p=0.9, min_p=0.05)}[case]
    pr, _ = host_ladder(logits[0].numpy(), p, [])
    kept = set(np.nonzero(pr)[0].tolist())
    assert 1 <= len(kept) < 200
    n = 400
    ids = s.sample(logits.repeat(n, 1).to(DEV), [p] * n, [9] * n, list(range(n)))
    assert set(ids) <= kept, sorted(set(ids) - kept)
    if len(kept) <= 12:
        assert set(ids) == kept            # with 400 draws every kept token of a small set appears


def test_penalties_and_bias_change_the_greedy_choice():
    from ultima_b200.sampling import SamplingParams
    V = 300
    s = _sampler(V)
    x = torch.zeros(1, V)
    x[0, 10], x[0, 20], x[0, 30] = 3.0, 2.9, 2.5
    assert s.sample(x.to(DEV), [SamplingParams()], [1], [0], [[]]) == [10]
    rep = SamplingParams(rep_penalty=1.2, repeat_last_n=8)
    assert s.sample(x.to(DEV), [rep], [1], [3], [[10, 10, 5]]) == [20]            # 3.0/1.2 < 2.9
    assert s.sample(x.to(DEV), [SamplingParams(rep_penalty=1.2, repeat_last_n=1)], [1], [3], [[10, 5]]) == [10]
    bias = SamplingParams(logit_bias={30: 1.0, 999: 5.0})
    assert s.sample(x.to(DEV), [bias], [1], [0], [[]]) == [30]
    fp = SamplingParams(frequency_penalty=0.3, presence_penalty=0.1, repeat_last_n=16)
    assert s.sample(x.to(DEV), [fp], [1], [2], [[10, 10]]) == [20]               # 3.0 - 0.6 - 0.1 < 2.9
    dry = SamplingParams(dry_multiplier=0.8, dry_base=1.75, dry_allowed_len=2, dry_last_n=32)
    assert s.sample(x.to(DEV), [dry], [1], [3], [[10, 10, 7]]) == [10]           # two repeats are allowed
    assert s.sample(x.to(DEV), [dry], [1], [4], [[10, 10, 10, 7]]) == [20]       # three are not
    for p, rec in ((rep, [10, 10, 5]), (fp, [10, 10]), (dry, [10, 10, 10, 7])):
        want, _ = host_ladder(x[0].numpy(), p, rec)
        assert s.sample(x.to(DEV), [p], [1], [len(rec)], [rec]) == [want]


@pytest.mark.parametrize("case", ["ties", "far_cut", "deep_top_p", "top_p_after_top_k", "wide_vocab"])
def test_cuts_on_rows_that_leave_the_fast_search(case):
    """Rows on which the three-pass search for the cut gives up (long runs of equal values, a cut
    further than 64 units below the maximum) or must be exact (a cumulative mass right at the
    boundary, top-p narrowing what top-k kept): the kept set is still the host's."""
    from ultima_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(21)
    if case == "ties":
        V = 6000
        logits = torch.zeros(1, V)
        logits[0, ::3] = 1.0                                   # 2,000 equal maxima: top-k keeps them all
        p = SamplingParams(temperature=1.0, top_k=5)
    elif case == "far_cut":
        V = 4000
        logits = torch.randn(1, V, generator=g) * 60           # the 500th largest lies far below the maximum
        p = SamplingParams(temperature=1.0, top_k=500)
    elif case == "deep_top_p":
        V = 9001
        logits = torch.randn(1, V, generator=g) * 0.05         # nearly flat: top-p keeps almost everything
        p = SamplingParams(temperature=1.0, top_p=0.97)
    elif case == "top_p_after_top_k":
        V = 3000
        logits = torch.randn(1, V, generator=g) * 2
        p = SamplingParams(temperature=1.0, top_k=64, top_p=0.5)
    else:
        V = 151936
        logits = torch.randn(1, V, generator=g) * 3
        p = SamplingParams(temperature=0.6, top_k=50, top_p=0.9, min_p=0.02)
    s = _sampler(V)
    pr, _ = host_ladder(logits[0].numpy(), p, [])
    kept = np.nonzero(pr)[0]
    n = 600
    ids = np.array(s.sample(logits.repeat(n, 1).to(DEV), [p] * n, [3] * n, list(range(n))))
    assert set(ids.tolist()) <= set(kept.tolist()), (case, sorted(set(ids.tolist()) - set(kept.tolist()))[:10])
    if case == "ties":
        assert len(kept) == 2000 and len(set(ids.tolist())) > 250          # spread over the tied maxima
    if case == "far_cut":
        assert len(kept) == 500
    if case == "deep_top_p":
        # the draws follow the kept distribution: low and high halves of the kept set by index
        # carry about the mass the host gives them
        half = kept[len(kept) // 2]
        host_low = pr[:half].sum()
        assert abs((ids < half).mean() - host_low) < 0.07
    if len(kept) <= 12:
        assert set(ids.tolist()) == set(kept.tolist())


def test_history_kept_on_the_device_follows_what_the_caller_holds():
    """The rings of recent tokens on the device give the same choices as sending the history with
    every call: a sequence that goes on (the kernel appends what it samples), a history that was
    edited behind the sampler's back, a new sequence under an old stream number, a long history
    that wraps the ring."""
    from ultima_b200.sampling import SamplingParams
    V = 400
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(3, V, generator=g) * 0.3).to(DEV)
    p = SamplingParams(rep_penalty=1.5, repeat_last_n=48, frequency_penalty=0.2, presence_penalty=0.1)
    s = _sampler(V)

    def fresh_choice(rows, hists):
        """What a sampler that has never seen these streams chooses."""
        return _sampler(V).sample(logits[rows], [p] * len(rows), [100 + r for r in rows], [0] * len(rows),
                                  [list(h) for h in hists])
    hists = [[1, 2, 3], [4], list(range(200, 330))]            # the third is longer than the ring
    streams = [11, 12, 13]
    for step in range(70):                                     # greedy with penalties never repeats for long
        got = s.sample(logits, [p] * 3, streams, [step] * 3, hists)
        assert got == fresh_choice([0, 1, 2], hists), step
        for h, t in zip(hists, got):
            h.append(t)
    # an edited history of the same length, and a new sequence under an old stream
    hists[0][-1] = (hists[0][-1] + 1) % V
    got = s.sample(logits, [p] * 3, streams, [70] * 3, hists)
    assert got == fresh_choice([0, 1, 2], hists)
    new = [[7, 7, 7, 8], [9]]
    got = s.sample(logits[:2], [p] * 2, streams[:2], [0, 0], new)
    assert got == fresh_choice([0, 1], new)
