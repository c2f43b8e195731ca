"""The layer-stack kernel (csrc/decode_stack.cu), which runs all layers of a decode step as one resident
kernel and is switched off unless asked for: switched on here, on the two tiny configurations with head
sizes 64 and 128, for batches of unequal lengths whose shorter requests leave, with a second batch in the
same slots; every logit against the plain implementation, and the kernel is seen to have run."""
import numpy as np
import pytest

from conftest import close_enough

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_seqs", [3, 19])
@pytest.mark.parametrize("name", ["D", "E"])
def test_layer_stack_kernel_gives_the_plain_logits(model_dirs, plain_models, monkeypatch, name, n_seqs):
    import plain_qwen3 as P
    from ultima_b200.engine import Engine
    from ultima_b200.kernels import decode_stack
    monkeypatch.setattr(decode_stack, "ENABLED", True)
    cfg, w = plain_models(name, "bfloat16")
    V, L = cfg["vocab_size"], cfg["num_hidden_layers"]
    eng = Engine.from_dir(model_dirs(name, "bfloat16"), dtype="bfloat16", max_tokens=n_seqs * 256, max_seqs=n_seqs,
                          poison_cache=True)
    rng = np.random.default_rng(77 + n_seqs)
    for b in range(2):
        plens = rng.integers(1, 100, size=n_seqs)
        dlens = rng.integers(2, 40, size=n_seqs)
        plens[0], dlens[0] = 60, 39                        # one sequence crosses a page edge while decoding
        seqs = [rng.integers(0, V, size=int(p + d)).tolist() for p, d in zip(plens, dlens)]
        slots = eng.open(n_seqs)
        out = eng.step(slots, [s[:p] for s, p in zip(seqs, plens)], [[int(p) - 1] for p in plens]).cpu().numpy()
        got = [{int(p) - 1: out[i]} for i, p in enumerate(plens)]
        live = list(range(n_seqs))
        t = 0
        while True:
            for i in [i for i in live if t >= dlens[i]]:
                eng.close([slots[i]])
                live.remove(i)
            if not live:
                break
            out = eng.step([slots[i] for i in live], [[seqs[i][plens[i] + t]] for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i][int(plens[i]) + t] = out[j]
            t += 1
        eng.check_errors()
        assert eng.cache.pages_held() == 0
        for i, ids in enumerate(seqs):
            ref = P.forward(cfg, w, ids)
            places = sorted(got[i])
            g_ = np.stack([got[i][pl] for pl in places])
            err, bound = close_enough(g_, ref[places], "bfloat16", L)
            assert err <= bound, f"[{name}] batch {b} request {i}: error {err:.3e} > {bound:.3e}"
    plan = eng.model._stack
    assert isinstance(plan, decode_stack.StackPlan) and plan.programs      # the decode steps went through the kernel
