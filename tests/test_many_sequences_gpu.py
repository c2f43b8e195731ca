"""Many sequences in a step: batches of 20, 33 and 64 prompts of unequal lengths, then decoding for 90
steps while the shorter requests leave, then a second batch in the same slots; on the two tiny
configurations whose head sizes (64, 128) send the bfloat16 path through the tcgen05 products with
token tiles of 32 and 64, the decode attention fed by TMA and its route straight from the projection's
slices.  Sequences grow across page edges, so the number of key slices of the decode attention changes
under way.  Every logit, in both element types, against the plain implementation."""
import numpy as np
import pytest

from conftest import close_enough

pytestmark = pytest.mark.gpu

_refs: dict = {}


def _plain(plain_models, name, ids):
    import plain_qwen3 as P
    key = (name, tuple(ids))
    if key not in _refs:
        cfg, w = plain_models(name, "bfloat16")
        _refs[key] = P.forward(cfg, w, ids)
    return _refs[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_seqs", [20, 33, 64])
@pytest.mark.parametrize("name", ["D", "E"])
def test_batches_of_many_unequal_sequences(model_dirs, plain_models, name, n_seqs, dtype):
    from ultima_b200.engine import Engine
    from ultima_b200.kernels import attn_tc
    cfg, _ = plain_models(name, "bfloat16")
    V, L = cfg["vocab_size"], cfg["num_hidden_layers"]
    eng = Engine.from_dir(model_dirs(name, "bfloat16"), dtype=dtype, max_tokens=n_seqs * 256, max_seqs=n_seqs,
                          poison_cache=True)
    rng = np.random.default_rng(1000 + n_seqs)
    slices_seen = set()
    for b in range(2):
        plens = rng.integers(1, 131, size=n_seqs)
        dlens = rng.integers(3, 91, size=n_seqs)
        dlens[0], plens[0] = 90, 130                       # one sequence goes all the way: four pages
        seqs = [rng.integers(0, V, size=int(p + d)).tolist() for p, d in zip(plens, dlens)]
        slots = eng.open(n_seqs)
        out = eng.step(slots, [s[:p] for s, p in zip(seqs, plens)], [[int(p) - 1] for p in plens]).cpu().numpy()
        got = [{int(p) - 1: out[i]} for i, p in enumerate(plens)]
        live = list(range(n_seqs))
        t = 0
        while True:
            for i in [i for i in live if t >= dlens[i]]:   # shorter requests end earlier
                eng.close([slots[i]])
                live.remove(i)
            if not live:
                break
            longest = max(int(plens[i]) + t + 1 for i in live)
            for g in eng.cache.kv_groups:
                slices_seen.add(attn_tc.decode_slices(len(live), g.need.n_kv_heads, longest, g.need.window))
            out = eng.step([slots[i] for i in live], [[seqs[i][plens[i] + t]] for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i][int(plens[i]) + t] = out[j]
            t += 1
        assert eng.cache.pages_held() == 0 and eng.cache.slots.n_free == n_seqs
        eng.check_errors()
        for i, ids in enumerate(seqs):
            ref = _plain(plain_models, name, ids)
            places = sorted(got[i])
            assert places == list(range(int(plens[i]) - 1, len(ids)))
            g_ = np.stack([got[i][pl] for pl in places])
            err, bound = close_enough(g_, ref[places], dtype, L)
            if err > bound:
                bad = places[int(np.argmax(np.abs(g_ - ref[places]).max(axis=1) > bound))]
                pytest.fail(f"[{name} {dtype} {n_seqs} sequences] batch {b} request {i} (prompt {plens[i]}, "
                            f"{len(ids)} tokens): error {err:.3e} > {bound:.3e}, first bad place {bad}")
    assert len(slices_seen) >= 2, slices_seen             # the key range was cut in different ways under way
