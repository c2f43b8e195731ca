"""Parts defined here, outside the package, registered and run through the engine without a change to
the package's files: a position encoding that is no rotation (called through ``Position.forward``
between the norm and the cache write), rotations of part of a head and of interleaved pairs, an
arrangement with other roles than the pre-norm block's, and a mixer with state of its own that allows
captured decode steps.  Each against a float64 restatement written beside it.  None of them is a
model of anyone's."""
import math

import numpy as np
import pytest
import torch

from conftest import random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rms(x, w, eps=1e-5):
    return x * w / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def _ffn(h, t, p):
    g, u = h @ t[p + "gate_proj.weight"].T, h @ t[p + "up_proj.weight"].T
    return (g / (1 + torch.exp(-g)) * u) @ t[p + "down_proj.weight"].T


def _attend(q, k, v, group, window=None):
    """q [n, nh, d], k, v [n, nkv, d] float64, causal."""
    n, nh, d = q.shape
    o = torch.zeros_like(q)
    for r in range(n):
        lo = max(0, r + 1 - window) if window else 0
        for h in range(nh):
            s = (k[lo:r + 1, h // group] @ q[r, h]) / math.sqrt(d)
            o[r, h] = torch.softmax(s, 0) @ v[lo:r + 1, h // group]
    return o


def _run_whole_then_one_by_one(eng, ids, cut):
    s = eng.open(1)
    got = [eng.step(s, [ids[:cut]], [list(range(cut))]).cpu().numpy()]
    for t in range(cut, len(ids)):
        got.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    return np.concatenate(got)


# ---------------------------------------------------------------------------------------
# a position encoding that is no rotation of pairs
# ---------------------------------------------------------------------------------------
def _register_decay_position():
    from ultima_b200.parts import Position, register_part

    @register_part("position", "toy_distance_decay", replace=True)
    class DistanceDecay(Position):
        """q_j *= s_j^pos, k_j *= s_j^(-pos) with s_j = exp(-rate * j / d): a score then carries
        s_j^(distance).  Not a rotation: ``rotation()`` stays None and the attention part calls
        ``forward`` between its norm kernel and the cache write."""

        def __init__(self, head_dim: int, rate: float, max_positions: int):
            self.head_dim, self.rate, self.max_positions = head_dim, rate, max_positions

        def bind(self, tensors, rt):
            j = torch.arange(self.head_dim, dtype=torch.float64)
            p = torch.arange(self.max_positions, dtype=torch.float64)
            e = -self.rate * p[:, None] * j[None] / self.head_dim
            self.up, self.down = torch.exp(e).float().to(rt.device), torch.exp(-e).float().to(rt.device)

        def forward(self, q, k, positions, rt):
            idx = positions.long()
            q.copy_((q.float() * self.up[idx][:, None, :]).to(q.dtype))
            k.copy_((k.float() * self.down[idx][:, None, :]).to(k.dtype))
    return DistanceDecay


def _tiny_spec(position, width=48, vocab=61, nh=4, nkv=2, hd=16, qk_norm=True, window=None):
    from ultima_b200.parts import ModelSpec, Run, layer, part
    norm = part("rms", width=width, eps=1e-5)
    att = part("attention", width=width, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm=qk_norm, eps=1e-5,
               position=position, window=window)
    layers = tuple(layer(part("pre_norm"), prefix=f"l{i}.", mixer=att, mixer_norm=norm, feed_forward_norm=norm,
                         feed_forward=part("gated_silu", width=width, inner=56)) for i in range(2))
    return ModelSpec(width=width, vocab_size=vocab, max_positions=128,
                     embedding=part("token_table", vocab_size=vocab, width=width), embedding_name="emb.",
                     layers=layers, runs=(Run(0), Run(1)), final_norm=norm, final_norm_name="fn.",
                     head=part("linear", vocab_size=vocab, width=width, tied=True), head_name="head.")


def _plain_attention_model(tensors, ids, encode, width=48, nh=4, nkv=2, hd=16, qk_norm=True, window=None):
    """Two pre-norm layers of attention and gated feed-forward in float64; ``encode(x, which)`` is the
    position encoding of x [n, heads, hd] (which: "q" or "k")."""
    t = {k: v.double().cpu() for k, v in tensors.items()}
    n = len(ids)
    x = t["emb.weight"][ids]
    for p in ("l0.", "l1."):
        h = _rms(x, t[p + "mixer_norm.weight"])
        q = (h @ t[p + "mixer.q_proj.weight"].T).view(n, nh, hd)
        k = (h @ t[p + "mixer.k_proj.weight"].T).view(n, nkv, hd)
        v = (h @ t[p + "mixer.v_proj.weight"].T).view(n, nkv, hd)
        if qk_norm:
            q, k = _rms(q, t[p + "mixer.q_norm.weight"]), _rms(k, t[p + "mixer.k_norm.weight"])
        o = _attend(encode(q, "q"), encode(k, "k"), v, nh // nkv, window)
        x = x + o.reshape(n, nh * hd) @ t[p + "mixer.o_proj.weight"].T
        x = x + _ffn(_rms(x, t[p + "feed_forward_norm.weight"]), t, p + "feed_forward.")
    return (_rms(x, t["fn.weight"]) @ t["emb.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_encoding_that_is_no_rotation_runs_through_forward(dtype):
    from ultima_b200.engine import Engine
    from ultima_b200.parts import part
    from ultima_b200.weights import random_tensors
    _register_decay_position()
    rate, hd = 0.6, 16
    spec = _tiny_spec(part("toy_distance_decay", head_dim=hd, rate=rate, max_positions=128), window=37)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.weight_specs(), 21, store).items()}
    eng = Engine(spec, tensors, dtype=dtype, max_tokens=512, max_seqs=2, poison_cache=True)
    assert not eng.use_graphs                          # the toy leaves graph_safe at its default

    def encode(x, which):
        n = x.shape[0]
        e = -rate * torch.arange(n, dtype=torch.float64)[:, None] * torch.arange(hd, dtype=torch.float64)[None] / hd
        return x * torch.exp(e if which == "q" else -e)[:, None, :]
    ids = random_ids(2, 70, 61)
    ref = _plain_attention_model(tensors, ids, encode, window=37)
    got = _run_whole_then_one_by_one(eng, ids, 45)
    tol = 3e-5 if dtype == "float32" else 4 * 2.0 ** -8
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("kind,rotary_dim", [("rotary_half_split", 8), ("rotary_interleaved", 16), ("rotary_interleaved", 12)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_of_part_of_a_head_and_of_interleaved_pairs(kind, rotary_dim, dtype):
    """The library's own rotary parts with fewer rotated columns than the head has, and with
    neighbouring columns as pairs: the kernels rotate while they norm and write the cache."""
    from ultima_b200.engine import Engine
    from ultima_b200.parts import part
    from ultima_b200.weights import random_tensors
    hd, theta = 16, 500.0
    spec = _tiny_spec(part(kind, head_dim=hd, theta=theta, max_positions=128, rotary_dim=rotary_dim))
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.weight_specs(), 22, store).items()}
    eng = Engine(spec, tensors, dtype=dtype, max_tokens=512, max_seqs=2, poison_cache=True)

    def encode(x, which):
        n, half = x.shape[0], rotary_dim // 2
        ang = torch.arange(n, dtype=torch.float64)[:, None] / torch.pow(
            torch.tensor(theta, dtype=torch.float64), 2.0 * torch.arange(half, dtype=torch.float64) / rotary_dim)[None]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        y = x.clone()
        if kind == "rotary_interleaved":
            a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
            y[..., 0:rotary_dim:2], y[..., 1:rotary_dim:2] = a * c - b * s, a * s + b * c
        else:
            a, b = x[..., :half], x[..., half:rotary_dim]
            y[..., :half], y[..., half:rotary_dim] = a * c - b * s, a * s + b * c
        return y
    ids = random_ids(3, 60, 61)
    ref = _plain_attention_model(tensors, ids, encode)
    got = _run_whole_then_one_by_one(eng, ids, 40)
    tol = 3e-5 if dtype == "float32" else 4 * 2.0 ** -8
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_rotary_forward_is_the_rotation_the_kernels_apply():
    """``Position.forward`` of the library's rotary parts (for mixers that call it themselves) against
    the same float64 rotation, on strided views."""
    from ultima_b200.engine import Runtime
    from ultima_b200.parts import build_part, part
    rt = Runtime(DEV, torch.float32)
    for kind, rd in (("rotary_half_split", 32), ("rotary_half_split", 20), ("rotary_interleaved", 32)):
        pos = build_part("position", part(kind, head_dim=32, theta=1e4, max_positions=300, rotary_dim=rd))
        pos.bind({}, rt)
        g = torch.Generator().manual_seed(rd)
        wide = torch.randn(7, 5 * 32 + 8, generator=g)
        q = wide.to(DEV)[:, :5 * 32].view(7, 5, 32)                  # rows of a wider matrix
        k = torch.randn(7, 2, 32, generator=g).to(DEV)
        q0, k0 = q.double().cpu(), k.double().cpu()
        positions = torch.tensor([0, 1, 5, 64, 65, 200, 299], dtype=torch.int32, device=DEV)
        pos.forward(q, k, positions, rt)
        half = rd // 2
        ang = positions.double().cpu()[:, None] / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                                                            2.0 * torch.arange(half, dtype=torch.float64) / rd)[None]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for got, x in ((q, q0), (k, k0)):
            y = x.clone()
            if kind == "rotary_interleaved":
                a, b = x[..., 0:rd:2], x[..., 1:rd:2]
                y[..., 0:rd:2], y[..., 1:rd:2] = a * c - b * s, a * s + b * c
            else:
                a, b = x[..., :half], x[..., half:rd]
                y[..., :half], y[..., half:rd] = a * c - b * s, a * s + b * c
            assert (got.double().cpu() - y).abs().max() < 2e-6, (kind, rd)


# ---------------------------------------------------------------------------------------
# an arrangement with roles of its own
# ---------------------------------------------------------------------------------------
def _register_parallel_arrangement():
    from ultima_b200.parts import Arrangement, register_part

    @register_part("arrangement", "toy_parallel", replace=True)
    class Parallel(Arrangement):
        """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, both branches read the same rows."""
        roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def __init__(self):
            pass

        def run(self, layer, x, batch, cache, rt):
            mark = rt.arena.mark()
            h = layer.norm.forward(x, rt)
            keep = rt.arena.mark()
            layer.mixer.forward(h, x, batch, cache, rt)
            rt.arena.reset(keep)
            layer.feed_forward.forward(h, x, batch, rt)
            rt.arena.reset(mark)
    return Parallel


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_arrangement_with_other_roles(dtype):
    from ultima_b200.engine import Engine
    from ultima_b200.parts import ModelSpec, Run, layer, part
    from ultima_b200.weights import random_tensors
    _register_parallel_arrangement()
    width, vocab, nh, nkv, hd = 64, 83, 4, 1, 16
    norm = part("rms", width=width, eps=1e-5)
    rot = part("rotary_half_split", head_dim=hd, theta=1e4, max_positions=128)
    att = part("attention", width=width, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qk_norm=False, eps=1e-5, position=rot)
    with pytest.raises(KeyError, match="no role 'mixer_norm'"):
        layer(part("toy_parallel"), mixer=att, feed_forward=part("gated_silu", width=width, inner=64), norm=norm,
              mixer_norm=norm)
    with pytest.raises(KeyError, match="needs a part in the role 'norm'"):
        layer(part("toy_parallel"), mixer=att, feed_forward=part("gated_silu", width=width, inner=64))
    layers = (layer(part("toy_parallel"), prefix="p0.", names={"norm": "ln."}, norm=norm, mixer=att,
                    feed_forward=part("gated_silu", width=width, inner=64)),
              layer(part("pre_norm"), prefix="p1.", mixer=att, mixer_norm=norm, feed_forward_norm=norm,
                    feed_forward=part("gated_silu", width=width, inner=96)))
    spec = ModelSpec(width=width, vocab_size=vocab, max_positions=128,
                     embedding=part("token_table", vocab_size=vocab, width=width), embedding_name="emb.",
                     layers=layers, runs=(Run(0), Run(1)), final_norm=norm, final_norm_name="fn.",
                     head=part("linear", vocab_size=vocab, width=width, tied=False), head_name="head.")
    names = [s.name for s in spec.weight_specs()]
    assert "p0.ln.weight" in names and "p0.mixer.q_proj.weight" in names and "p0.mixer_norm.weight" not in names
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.weight_specs(), 23, store).items()}
    eng = Engine(spec, tensors, dtype=dtype, max_tokens=512, max_seqs=2, poison_cache=True)
    assert eng.use_graphs                              # only library parts and a toy arrangement: decode steps are captured

    def plain(ids):
        t = {k: v.double().cpu() for k, v in tensors.items()}
        n = len(ids)
        x = t["emb.weight"][ids]
        half = hd // 2
        ang = torch.arange(n, dtype=torch.float64)[:, None] / torch.pow(
            torch.tensor(1e4, dtype=torch.float64), 2.0 * torch.arange(half, dtype=torch.float64) / hd)[None]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        rot_ = lambda v: torch.cat([v[..., :half] * c - v[..., half:] * s, v[..., :half] * s + v[..., half:] * c], -1)

        def att_(h, p):
            q = rot_((h @ t[p + "q_proj.weight"].T).view(n, nh, hd))
            k = rot_((h @ t[p + "k_proj.weight"].T).view(n, nkv, hd))
            v = (h @ t[p + "v_proj.weight"].T).view(n, nkv, hd)
            return _attend(q, k, v, nh // nkv).reshape(n, nh * hd) @ t[p + "o_proj.weight"].T
        h = _rms(x, t["p0.ln.weight"])
        x = x + att_(h, "p0.mixer.") + _ffn(h, t, "p0.feed_forward.")
        x = x + att_(_rms(x, t["p1.mixer_norm.weight"]), "p1.mixer.")
        x = x + _ffn(_rms(x, t["p1.feed_forward_norm.weight"]), t, "p1.feed_forward.")
        return (_rms(x, t["fn.weight"]) @ t["head.weight"].T).numpy()
    ids = random_ids(5, 50, vocab)
    ref = plain(ids)
    got = _run_whole_then_one_by_one(eng, ids, 30)
    tol = 3e-5 if dtype == "float32" else 4 * 2.0 ** -8
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


# ---------------------------------------------------------------------------------------
# a mixer with state of its own whose decode steps may be captured
# ---------------------------------------------------------------------------------------
def _register_capturable_state_mixer():
    from ultima_b200.parts import Mixer, StateNeed, register_part
    from ultima_b200.weights import WeightSpec

    @register_part("mixer", "toy_running_mean_on_device", replace=True)
    class RunningMeanOnDevice(Mixer):
        """state <- decay * state + (1 - decay) * h_t; out_t = W state.  A step of one token a sequence
        touches the state with device work only (rows picked by the step record's slot numbers), so
        it says graph_safe; prompts go token by token from the host's lengths, which are not captured."""
        graph_safe = True

        def __init__(self, width: int, decay: float):
            self.width, self.decay = width, decay

        def weight_specs(self):
            return [WeightSpec("mix.weight", (self.width, self.width), "matrix", ("normal", 0.2))]

        def cache_need(self):
            return StateNeed((self.width,), "float32")

        def bind(self, tensors, rt):
            self.w = tensors["mix.weight"].float()

        def forward(self, h, residual, batch, cache, rt):
            if batch.max_new == 1:
                idx = batch.seq_slot.long()
                st = cache.state[idx] * self.decay + h.float() * (1 - self.decay)
                cache.state.index_copy_(0, idx, st)
                residual.add_(st @ self.w.T)
                return
            lens, slots = batch.host["lens"], batch.seq_slot.tolist()
            row = 0
            for s, n in zip(slots, lens):
                st = cache.state[s]
                for t in range(int(n)):
                    st.mul_(self.decay).add_(h[row + t].float(), alpha=1 - self.decay)
                    residual[row + t] += self.w @ st
                row += int(n)
    return RunningMeanOnDevice


def test_state_of_a_capturable_mixer_advances_once_a_step():
    """Every new number of sequences makes the engine capture a new graph; the step that is captured
    must still run exactly once.  Sequences end one after another, so the batch shrinks 4, 3, 2, 1 and
    four graphs are made; a state that advanced twice anywhere would show in every logit after."""
    from ultima_b200.engine import Engine
    from ultima_b200.parts import ModelSpec, Run, layer, part
    from ultima_b200.weights import random_tensors
    _register_capturable_state_mixer()
    width, vocab, decay = 40, 97, 0.8
    norm = part("rms", width=width, eps=1e-5)
    layers = (layer(part("pre_norm"), prefix="l0.", mixer=part("toy_running_mean_on_device", width=width, decay=decay),
                    feed_forward=part("gated_silu", width=width, inner=56), mixer_norm=norm, feed_forward_norm=norm),)
    spec = ModelSpec(width=width, vocab_size=vocab, max_positions=256,
                     embedding=part("token_table", vocab_size=vocab, width=width), embedding_name="emb.",
                     layers=layers, runs=(Run(0),), final_norm=norm, final_norm_name="out_norm.",
                     head=part("linear", vocab_size=vocab, width=width, tied=False), head_name="head.")
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.weight_specs(), 4).items()}
    eng = Engine(spec, tensors, dtype="float32", max_tokens=1024, max_seqs=4)
    assert eng.use_graphs

    def plain(ids):
        t = {k: v.double().cpu() for k, v in tensors.items()}
        x = t["emb.weight"][ids]
        h = _rms(x, t["l0.mixer_norm.weight"])
        st, rows = torch.zeros(width, dtype=torch.float64), []
        for r in range(len(ids)):
            st = decay * st + (1 - decay) * h[r]
            rows.append(st)
        x = x + torch.stack(rows) @ t["l0.mixer.mix.weight"].T
        x = x + _ffn(_rms(x, t["l0.feed_forward_norm.weight"]), t, "l0.feed_forward.")
        return (_rms(x, t["out_norm.weight"]) @ t["head.weight"].T).numpy()
    seqs = [random_ids(10 + i, n, vocab) for i, n in enumerate((30, 24, 18, 12))]
    cut = [6, 5, 4, 3]
    refs = [plain(s) for s in seqs]
    for round_ in range(2):                            # the second round replays the graphs of the first
        slots = eng.open(4)
        out = eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
        got, o = [], 0
        for c in cut:
            got.append([out[o:o + c]])
            o += c
        live, t = [0, 1, 2, 3], 0
        while True:
            live = [i for i in live if cut[i] + t < len(seqs[i])]
            if not live:
                break
            out = eng.step([slots[i] for i in live], [[seqs[i][cut[i] + t]] for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            t += 1
        eng.close(slots)
        assert len(eng._graphs) == 4
        for i in range(4):
            err = np.abs(np.concatenate(got[i]) - refs[i]).max()
            assert err < 3e-5, (round_, i, err)
