"""The counter-based generator of random weights: the package's numpy version against the tests' own
copy (scalar and array forms), bit for bit, in float32 and after rounding to bfloat16; the
distribution; independence from the order and the other tensors; the written folder."""
import numpy as np
import torch

import plain_random as R
from conftest import TINY


def test_package_and_test_copies_agree_bit_for_bit():
    from ultima_b200.weights import counter_normal
    for key in (0, 1, R.tensor_key(7, "model.layers.0.self_attn.q_proj.weight"), (1 << 63) - 1):
        a = counter_normal(key, 0, 5000)
        b = R.normal_array(key, 5000)
        assert a.dtype == np.float32 and (a.view(np.uint32) == b.view(np.uint32)).all()
        for i in (0, 1, 2, 77, 4999):
            one = R.normal_one(key, i)
            assert np.float32(one).view(np.uint32) == a[i:i + 1].view(np.uint32)[0], (key, i)
        # a range that does not begin at zero gives the same elements
        c = counter_normal(key, 1234, 100)
        assert (c.view(np.uint32) == a[1234:1334].view(np.uint32)).all()


def test_the_draws_look_normal():
    from ultima_b200.weights import counter_normal
    z = counter_normal(42, 0, 400000).astype(np.float64)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    assert abs(np.mean(z ** 3)) < 0.03 and abs(np.mean(z ** 4) - 3.0) < 0.06
    assert 0.66 < np.mean(np.abs(z) < 1.0) < 0.70 and np.abs(z).max() > 4.0
    assert np.isfinite(z).all()
    # neighbours are not correlated
    assert abs(np.corrcoef(z[:-1], z[1:])[0, 1]) < 0.01


def test_random_tensors_are_the_generator_by_name():
    import ultima_b200 as u
    from ultima_b200.weights import random_tensors
    cfg = u.config_from_dict(TINY["B"])
    specs = u.model_spec_for(cfg).weight_specs()
    for dtype, name in ((torch.float32, "float32"), (torch.bfloat16, "bfloat16")):
        got = random_tensors(specs, 7, dtype)
        for s in specs[:6] + specs[-2:]:
            want = R.tensor(7, s.name, s.shape, s.init, name)
            have = got[s.name].float().numpy()
            assert have.shape == tuple(s.shape)
            assert (have.view(np.uint32) == want.view(np.uint32)).all(), (s.name, name)
    # a tensor's values do not depend on which other tensors are drawn with it
    alone = random_tensors([specs[3]], 7)
    assert torch.equal(alone[specs[3].name], random_tensors(specs, 7)[specs[3].name])
    assert not torch.equal(alone[specs[3].name], random_tensors([specs[3]], 8)[specs[3].name])


def test_written_folder_holds_those_values(tmp_path):
    import plain_qwen3 as P
    import ultima_b200 as u
    cfg = u.config_from_dict(TINY["A"])
    d = u.write_random_model(str(tmp_path / "m"), cfg, 3, "bfloat16")
    _, w = P.read_folder(d)
    spec = {s.name: s for s in u.model_spec_for(cfg).weight_specs()}
    for name in ("model.embed_tokens.weight", "model.layers.1.mlp.down_proj.weight", "model.norm.weight"):
        want = R.tensor(3, name, spec[name].shape, spec[name].init, "bfloat16")
        assert (w[name].astype(np.float32).view(np.uint32) == want.view(np.uint32)).all(), name
