"""The plain implementation against the reference's own model code (no GPU).

tests/golden/tiny_{A,B,C}.npz hold the logits that tattooinmtl/Ultima.cpp's model code, compiled
unchanged for the CPU by tests/golden/make_golden.py, gives on three tiny Qwen3 models whose
weights come from integer arithmetic (tests/golden/golden_weights.py); the third has a sliding
window of 4 positions on two of its three layers, which pins the window's edge (p - window, p] and
its per-layer pattern to the reference's own code.  The reference computes
in float32, the plain implementation in float64; they agree to float32 rounding.  The reference's
whole-prompt logits equal its token-by-token logits exactly, which the files record too."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import golden_weights as G  # noqa: E402
import plain_qwen3 as P  # noqa: E402


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_matches_the_reference(name):
    gold = np.load(os.path.join(HERE, "golden", f"tiny_{name}.npz"))
    cfg = G.CONFIGS[name]
    w = {k: v.astype(np.float64) for k, v in G.weights(cfg).items()}
    ids = G.PROMPTS[name]
    logits = P.forward(cfg, w, ids)
    ref = gold["decode_logits"].astype(np.float64)
    got = logits[gold["positions"]]
    assert np.abs(ref).max() > 1.0                        # the comparison is not between flat zeros
    assert np.abs(got - ref).max() < 2e-6, np.abs(got - ref).max()
    assert np.abs(logits[-1] - gold["prefill_last_logits"]).max() < 2e-6
    assert float(gold["prefill_vs_decode_max_abs"]) == 0.0
    # greedy: the reference's first-maximum rule picks the same token at every kept position
    for r, g in zip(ref, got):
        assert int(np.argmax(r)) == P.argmax_first(g)
