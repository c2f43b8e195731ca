"""The kernels at the layer sizes of a real checkpoint (Qwen3-8B: width 4096, 32 query and 8 KV
heads of 128, inner width 12288, vocabulary 151936), two layers, random weights: the bfloat16
path (tcgen05 products with every token tile, tensor-core attention with several key slices,
captured decode steps) against the 32-bit path of the same engine on the same weights, whole
prompts, a continued prompt and decoding past several pages."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
             intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
             head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=4096,
             tie_word_embeddings=False, hidden_act="silu")


@pytest.fixture(scope="module")
def engines():
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.weights import random_tensors_on_device
    cfg = u.config_from_dict(SIZES)
    spec = u.model_spec_for(cfg)
    t16 = random_tensors_on_device(spec.weight_specs(), 5, torch.bfloat16, "cuda:0")
    t32 = {k: v.float() for k, v in t16.items()}
    e16 = Engine(spec, t16, dtype="bfloat16", max_tokens=8192, max_seqs=8, max_step_tokens=1024)
    e32 = Engine(spec, t32, dtype="float32", max_tokens=8192, max_seqs=8, max_step_tokens=1024)
    return e16, e32, cfg.vocab_size


def _run(eng, prompts, decode, want_last_only=True):
    """Prompts in one step, then ``decode`` given tokens each, one a step; logits of every step's
    last places."""
    slots = eng.open(len(prompts))
    rows = [eng.step(slots, prompts, None).float().cpu().numpy()]
    for t in range(len(decode[0])):
        rows.append(eng.step(slots, [[d[t]] for d in decode], None).float().cpu().numpy())
    eng.close(slots)
    return np.stack(rows)            # [steps, sequences, vocabulary]


def test_bfloat16_path_agrees_with_the_32_bit_path_at_real_sizes(engines):
    e16, e32, V = engines
    rng = np.random.default_rng(0)
    lens = [1, 300, 777, 130]                       # token tiles of 16 ... 256 and several passes
    prompts = [rng.integers(0, V, size=n).tolist() for n in lens]
    decode = [rng.integers(0, V, size=6).tolist() for _ in lens]
    a, b = _run(e16, prompts, decode), _run(e32, prompts, decode)
    assert np.isfinite(a).all() and np.isfinite(b).all()
    scale = np.abs(b).max()
    err = np.abs(a - b).max()
    # two layers of bfloat16 activations: a few times 2^-8 of the largest logit
    assert err <= 4 * 2.0 ** -8 * scale, (err, scale)
    # and the two paths choose the same token wherever the 32-bit choice is clear
    top2 = np.sort(b, axis=-1)[..., -2:]
    clear = (top2[..., 1] - top2[..., 0]) > 8 * 2.0 ** -8 * scale
    assert clear.any()
    assert (a.argmax(-1)[clear] == b.argmax(-1)[clear]).all()


def test_decode_far_into_the_context_with_key_slices(engines):
    e16, e32, V = engines
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, V, size=2100).tolist()]          # one sequence: the key range is sliced
    decode = [rng.integers(0, V, size=4).tolist()]
    a, b = _run(e16, prompts, decode), _run(e32, prompts, decode)
    scale = np.abs(b).max()
    assert np.abs(a - b).max() <= 4 * 2.0 ** -8 * scale
    e16.check_errors()
    e32.check_errors()
