"""Each part alone against the plain functions; a run list that names a layer twice and lets a
run read another run's cache; and a toy mixer with state of its own, defined here, registered,
built and stepped without a change to the package's files."""
import math

import numpy as np
import pytest
import torch

from conftest import TINY, random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rt(dtype=torch.float32):
    from ultima_b200.engine import Runtime
    return Runtime(DEV, dtype)


def _batch(slots, new, before, want, tables):
    from ultima_b200.engine import build_step_batch
    return build_step_batch(slots, new, before, want, tables, torch.device(DEV))


def test_norm_part():
    import plain_qwen3 as P
    from ultima_b200.parts import build_part, part
    rt = _rt()
    n = build_part("norm", part("rms", width=75, eps=1e-4))
    assert [(s.name, s.shape, s.kind) for s in n.weight_specs()] == [("weight", (75,), "vector")]
    w = torch.randn(75) * 0.1 + 1
    n.bind({"weight": w.to(DEV)}, rt)
    x = torch.randn(6, 75)
    got = n.forward(x.to(DEV), rt).cpu().numpy()
    assert np.abs(got - P.rmsnorm(x.double().numpy(), w.double().numpy(), 1e-4)).max() < 2e-6


def test_position_part_tables_are_shared():
    from ultima_b200.parts import build_part, part
    rt = _rt()
    spec = part("rotary_half_split", head_dim=48, theta=5e5, max_positions=300)
    a, b = build_part("position", spec), build_part("position", spec)
    a.bind({}, rt)
    b.bind({}, rt)
    assert a.cos.data_ptr() == b.cos.data_ptr() and a.cos.shape == (300, 24)
    j = np.arange(24)
    ang = 299 * (1.0 / np.power(5e5, 2.0 * j / 48))
    assert np.abs(a.cos[299].cpu().numpy() - np.cos(ang)).max() < 1e-6
    assert np.abs(a.sin[299].cpu().numpy() - np.sin(ang)).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone(dtype):
    """One attention part, a cache made by hand, a prompt in one step and two more tokens."""
    import plain_qwen3 as P
    from ultima_b200.cache import Cache
    from ultima_b200.parts import build_part, part
    rt = _rt(dtype)
    width, nh, nkv, hd, eps, theta, window = 72, 6, 2, 32, 1e-5, 1e4, 9
    pos = part("rotary_half_split", head_dim=hd, theta=theta, max_positions=128)
    att = build_part("mixer", part("attention", width=width, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                                   qk_norm=True, eps=eps, position=pos, window=window))
    g = torch.Generator().manual_seed(0)
    tens = {}
    for s in att.weight_specs():
        t = torch.randn(s.shape, generator=g) * (0.1 if s.kind == "matrix" else 0.05)
        tens[s.name] = (t + (1 if s.kind == "vector" else 0)).to(dtype if s.kind == "matrix" else torch.float32)
    att.bind({k: v.to(DEV) for k, v in tens.items()}, rt)
    cache = Cache([att.cache_need()], [None], max_tokens=256, max_context=128, n_slots=2, step_chunk=64,
                  dtype=dtype, device=DEV, poison=True)
    n = 20
    h = (torch.randn(n, width, generator=g)).to(dtype)
    w64 = {"x." + k: v.double().numpy() for k, v in tens.items()}
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rms_norm_eps=eps, rope_theta=theta)
    ref = P.attention_part(h.double().numpy(), w64, "x.", cfg, np.arange(n), window)
    slot = cache.acquire()
    got = []
    for lo, hi in ((0, 18), (18, 19), (19, 20)):
        cache.reserve(slot, hi)
        b = _batch([slot], [[0] * (hi - lo)], [lo], [], cache.tables([slot]))
        res = torch.zeros(hi - lo, width, device=DEV)
        rt.arena.reset()
        att.forward(h[lo:hi].to(DEV).contiguous(), res, b, cache.run_cache(0, b.tables), rt)
        cache.commit(slot, hi - lo)
        got.append(res.cpu().numpy())
    got = np.concatenate(got)
    tol = 1e-5 if dtype == torch.float32 else 0.05
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part_alone(dtype):
    import plain_qwen3 as P
    from ultima_b200.parts import build_part, part
    rt = _rt(dtype)
    ff = build_part("feed_forward", part("gated_silu", width=72, inner=200))
    g = torch.Generator().manual_seed(1)
    tens = {s.name: (torch.randn(s.shape, generator=g) * 0.1).to(dtype) for s in ff.weight_specs()}
    ff.bind({k: v.to(DEV) for k, v in tens.items()}, rt)
    h = torch.randn(9, 72, generator=g).to(dtype)
    res = torch.ones(9, 72, device=DEV)
    ff.forward(h.to(DEV), res, None, rt)
    ref = 1 + P.mlp_part(h.double().numpy(), {"m." + k: v.double().numpy() for k, v in tens.items()}, "m.")
    tol = 1e-5 if dtype == torch.float32 else 0.03
    assert np.abs(res.cpu().numpy() - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_embedding_and_head_parts():
    from ultima_b200.parts import build_part, part
    rt = _rt()
    emb = build_part("embedding", part("token_table", vocab_size=50, width=24))
    table = torch.randn(50, 24)
    emb.bind({"weight": table.to(DEV)}, rt)
    ids = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids, rt).cpu(), table[[3, 49, 0]])
    head = build_part("head", part("linear", vocab_size=50, width=24, tied=True))
    assert head.weight_specs() == []
    head.bind({"weight": emb.table}, rt)
    h = torch.randn(2, 24)
    got = head.forward(h.to(DEV), rt).cpu()
    assert got.dtype == torch.float32 and (got - h @ table.T).abs().max() < 1e-5


def test_run_list_names_a_layer_twice_and_shares_a_cache(model_dirs, plain_models):
    """Runs: layer 0, layer 1, layer 0 again (a cache of its own), layer 1 reading the cache of
    the second run.  Whole prompt, then token by token; both against a plain restatement."""
    import dataclasses
    import plain_qwen3 as P
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.parts import Run
    from ultima_b200.weights import load_weights
    name = "A"
    cfg_d, w = plain_models(name, "float32")
    cfg = u.config_from_dict(TINY[name])
    spec = u.model_spec_for(cfg)
    spec = dataclasses.replace(spec, runs=(Run(0), Run(1), Run(0), Run(1, cache_from=1)))
    tensors = load_weights(model_dirs(name, "float32"), spec.weight_specs(), torch.float32, DEV)
    eng = Engine(spec, tensors, dtype="float32", max_tokens=512, poison_cache=True)
    assert [g.runs for g in eng.cache.kv_groups] == [[0, 1, 2]]

    def plain(ids):
        n = len(ids)
        pos = np.arange(n)
        eps = cfg_d["rms_norm_eps"]
        nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        x = P.embed(w["model.embed_tokens.weight"], ids)
        kept = {}
        for r, (layer, src) in enumerate(((0, None), (1, None), (0, None), (1, 1))):
            p = f"model.layers.{layer}."
            h = P.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
            a = p + "self_attn."
            q = P.rope_half_split(P.rmsnorm(P.linear(h, w[a + "q_proj.weight"]).reshape(n, nh, d),
                                            w[a + "q_norm.weight"], eps), pos, cfg.rope_theta)
            if src is None:
                k = P.rope_half_split(P.rmsnorm(P.linear(h, w[a + "k_proj.weight"]).reshape(n, nkv, d),
                                                w[a + "k_norm.weight"], eps), pos, cfg.rope_theta)
                v = P.linear(h, w[a + "v_proj.weight"]).reshape(n, nkv, d)
                kept[r] = (k, v)
            else:
                k, v = kept[src]
            o = P.attention(q, k, v, pos).reshape(n, nh * d)
            x = x + P.linear(o, w[a + "o_proj.weight"])
            h = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
            x = x + P.mlp_part(h, w, p + "mlp.")
        h = P.rmsnorm(x, w["model.norm.weight"], eps)
        return P.linear(h, w["model.embed_tokens.weight"])

    ids = random_ids(8, 40, cfg.vocab_size)
    ref = plain(ids)
    s = eng.open(1)
    got = [eng.step(s, [ids[:30]], [list(range(30))]).cpu().numpy()]
    for t in range(30, 40):
        got.append(eng.step(s, [[ids[t]]], [[0]]).cpu().numpy())
    eng.close(s)
    assert np.abs(np.concatenate(got) - ref).max() < 2e-5


# ---------------------------------------------------------------------------------------
# a toy mixer with state of its own
# ---------------------------------------------------------------------------------------
def _register_toy():
    from ultima_b200.parts import Mixer, StateNeed, register_part
    from ultima_b200.weights import WeightSpec
    from ultima_b200.kernels import ops

    @register_part("mixer", "toy_running_mean", replace=True)
    class RunningMean(Mixer):
        """state <- decay * state + (1 - decay) * h_t;  out_t = W state.  Tokens of a sequence
        go in order; the state lives in the cache's fixed-size area, one row a slot."""

        def __init__(self, width: int, decay: float):
            self.width, self.decay = width, decay

        def weight_specs(self):
            return [WeightSpec("mix.weight", (self.width, self.width), "matrix", ("normal", 0.2))]

        def cache_need(self):
            return StateNeed((self.width,), "float32")

        def bind(self, tensors, rt):
            self.w = tensors["mix.weight"].float()

        def forward(self, h, residual, batch, cache, rt):
            lens, slots = batch.host["lens"], batch.seq_slot.tolist()
            row = 0
            states = torch.empty(h.shape[0], self.width, device=h.device)
            for s, n in zip(slots, lens):
                st = cache.state[s]
                for t in range(int(n)):
                    st.mul_(self.decay).add_(h[row + t].float(), alpha=1 - self.decay)
                    states[row + t] = st
                row += int(n)
            out = torch.empty(h.shape[0], self.width, device=h.device)
            ops.gemm_simt(states, self.w, out)
            ops.add_into(residual, out)
    return RunningMean


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from ultima_b200.engine import Engine
    from ultima_b200.parts import ModelSpec, Run, layer, part
    from ultima_b200.weights import random_tensors
    _register_toy()
    width, vocab, decay = 40, 97, 0.75
    norm = part("rms", width=width, eps=1e-5)
    att = part("attention", width=width, n_heads=2, n_kv_heads=1, head_dim=16, qk_norm=False, eps=1e-5,
               position=None, window=None)
    layers = (
        layer(part("pre_norm"), prefix="l0.", mixer=part("toy_running_mean", width=width, decay=decay),
              feed_forward=part("gated_silu", width=width, inner=56), mixer_norm=norm, feed_forward_norm=norm),
        layer(part("pre_norm"), prefix="l1.", mixer=att, feed_forward=part("gated_silu", width=width, inner=72),
              mixer_norm=norm, feed_forward_norm=norm),
        layer(part("pre_norm"), prefix="l2.", mixer=part("toy_running_mean", width=width, decay=0.5),
              feed_forward=part("gated_silu", width=width, inner=56), mixer_norm=norm, feed_forward_norm=norm),
    )
    spec = ModelSpec(width=width, vocab_size=vocab, max_positions=256,
                     embedding=part("token_table", vocab_size=vocab, width=width), embedding_name="emb.",
                     layers=layers, runs=(Run(0), Run(1), Run(2)), final_norm=norm, final_norm_name="out_norm.",
                     head=part("linear", vocab_size=vocab, width=width, tied=False), head_name="head.")
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.weight_specs(), 3).items()}
    eng = Engine(spec, tensors, dtype="float32", max_tokens=1024, max_seqs=3, poison_cache=True)
    # the two toy runs ask for the same state shape and share one state group; attention has its pages
    assert len(eng.cache.state_groups) == 1 and eng.cache.state_groups[0].runs == [0, 2]
    assert eng.cache.state_groups[0].data.shape == (2, 3, width) and len(eng.cache.kv_groups) == 1

    def plain(ids):
        """Whole sequence in float64 torch, state carried along."""
        t = {k: v.double().cpu() for k, v in tensors.items()}
        x = t["emb.weight"][ids]
        def rms(x, w):
            return x * w / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)
        def ffn(h, p):
            g, u_ = h @ t[p + "gate_proj.weight"].T, h @ t[p + "up_proj.weight"].T
            return (g / (1 + torch.exp(-g)) * u_) @ t[p + "down_proj.weight"].T
        for li, (kind, d) in enumerate((("toy", decay), ("att", None), ("toy", 0.5))):
            p = f"l{li}."
            h = rms(x, t[p + "mixer_norm.weight"])
            if kind == "toy":
                st = torch.zeros(width, dtype=torch.float64)
                rows = []
                for r in range(len(ids)):
                    st = d * st + (1 - d) * h[r]
                    rows.append(st)
                x = x + torch.stack(rows) @ t[p + "mixer.mix.weight"].T
            else:
                n = len(ids)
                q = (h @ t[p + "mixer.q_proj.weight"].T).view(n, 2, 16)
                k = (h @ t[p + "mixer.k_proj.weight"].T).view(n, 1, 16)
                v = (h @ t[p + "mixer.v_proj.weight"].T).view(n, 1, 16)
                o = torch.zeros(n, 2, 16, dtype=torch.float64)
                for r in range(n):
                    for hh in range(2):
                        s = (k[:r + 1, 0] @ q[r, hh]) / 4.0
                        o[r, hh] = torch.softmax(s, 0) @ v[:r + 1, 0]
                x = x + o.view(n, 32) @ t[p + "mixer.o_proj.weight"].T
            x = x + ffn(rms(x, t[p + "feed_forward_norm.weight"]), p + "feed_forward.")
        return (rms(x, t["out_norm.weight"]) @ t["head.weight"].T).numpy()

    seqs = [random_ids(i, n, vocab) for i, n in enumerate((70, 9, 33))]
    refs = [plain(s) for s in seqs]
    # a batch of unequal prompts, then token by token; the shortest ends first; then the slots are
    # used again by a second batch, whose state must start at zero
    for round_ in range(2):
        slots = eng.open(3)
        cut = [40, 4, 20]
        out = eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
        got, o = [], 0
        for c in cut:
            got.append([out[o:o + c]])
            o += c
        live = [0, 1, 2]
        t = 0
        while live:
            live = [i for i in live if cut[i] + t < len(seqs[i])]
            if not live:
                break
            out = eng.step([slots[i] for i in live], [[seqs[i][cut[i] + t]] for i in live], [[0]] * len(live))
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1].cpu().numpy())
            t += 1
        eng.close(slots)
        for i in range(3):
            assert np.abs(np.concatenate(got[i]) - refs[i]).max() < 3e-5, (round_, i)


# ---------------------------------------------------------------------------------------
# toy parts of the other families, defined here: a feed-forward with routing, another position
# encoding; they never become a model of anyone's
# ---------------------------------------------------------------------------------------
def _register_toy_routed_ffn():
    from ultima_b200.parts import FeedForward, register_part
    from ultima_b200.weights import WeightSpec
    from ultima_b200.kernels import ops

    @register_part("feed_forward", "toy_top1_experts", replace=True)
    class Top1Experts(FeedForward):
        """A router picks one of ``n_experts`` small gated feed-forwards for every token (router
        logits in float32); tokens are grouped by expert on the host and each group runs the
        library's products."""

        def __init__(self, width: int, inner: int, n_experts: int):
            self.width, self.inner, self.n = width, inner, n_experts

        def weight_specs(self):
            s = [WeightSpec("router.weight", (self.n, self.width), "matrix", ("normal", 0.5))]
            for e in range(self.n):
                s += [WeightSpec(f"experts.{e}.gate.weight", (self.inner, self.width), "matrix", ("normal", 0.2)),
                      WeightSpec(f"experts.{e}.up.weight", (self.inner, self.width), "matrix", ("normal", 0.2)),
                      WeightSpec(f"experts.{e}.down.weight", (self.width, self.inner), "matrix", ("normal", 0.2))]
            return s

        def bind(self, tensors, rt):
            self.router = tensors["router.weight"].float().contiguous()
            self.experts = [(tensors[f"experts.{e}.gate.weight"].contiguous(), tensors[f"experts.{e}.up.weight"].contiguous(),
                             tensors[f"experts.{e}.down.weight"].contiguous()) for e in range(self.n)]

        def forward(self, h, residual, batch, rt):
            T = h.shape[0]
            logits = torch.empty(T, self.n, dtype=torch.float32, device=h.device)
            ops.gemm_simt(h.float().contiguous(), self.router, logits)           # router in 32-bit
            choice = logits.argmax(-1)
            for e, (g, u, d) in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                x = h[rows].contiguous()
                a = torch.empty(rows.numel(), self.inner, dtype=h.dtype, device=h.device)
                ops.gemm_simt(x, g, a, ops.EPI_SWIGLU, w2=u)
                y = torch.zeros(rows.numel(), self.width, dtype=torch.float32, device=h.device)
                ops.gemm_simt(a, d, y, ops.EPI_ADD)
                residual.index_add_(0, rows, y)
    return Top1Experts


def _register_toy_position():
    from ultima_b200.parts import Position, Rotation, register_part

    @register_part("position", "toy_slow_rotary", replace=True)
    class SlowRotary(Position):
        """Half-split rotation with angle pos * scale / (j + 1): other tables, described to the
        attention part as a rotation, so the library's kernels apply it."""

        def __init__(self, head_dim: int, scale: float, max_positions: int):
            self.head_dim, self.scale, self.max_positions = head_dim, scale, max_positions
            self.cos = self.sin = None

        def bind(self, tensors, rt):
            half = self.head_dim // 2
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * self.scale / \
                (torch.arange(half, dtype=torch.float64)[None] + 1)
            self.cos, self.sin = torch.cos(ang).float().to(rt.device), torch.sin(ang).float().to(rt.device)

        def rotation(self):
            return Rotation(self.cos, self.sin, self.head_dim, False)
    return SlowRotary


def test_toy_routed_feed_forward_and_another_position_encoding():
    from ultima_b200.engine import Engine
    from ultima_b200.parts import ModelSpec, Run, layer, part
    from ultima_b200.weights import random_tensors
    _register_toy_routed_ffn()
    _register_toy_position()
    width, vocab, hd, n_exp = 48, 61, 16, 3
    norm = part("rms", width=width, eps=1e-5)
    pos = part("toy_slow_rotary", head_dim=hd, scale=0.3, max_positions=128)
    att = part("attention", width=width, n_heads=3, n_kv_heads=3, head_dim=hd, qk_norm=True, eps=1e-5, position=pos)
    layers = (layer(part("pre_norm"), prefix="a.", mixer=att, mixer_norm=norm, feed_forward_norm=norm,
                    feed_forward=part("toy_top1_experts", width=width, inner=40, n_experts=n_exp)),
              layer(part("pre_norm"), prefix="b.", mixer=att, mixer_norm=norm, feed_forward_norm=norm,
                    feed_forward=part("gated_silu", width=width, inner=64)))
    spec = ModelSpec(width=width, vocab_size=vocab, max_positions=128,
                     embedding=part("token_table", vocab_size=vocab, width=width), embedding_name="emb.",
                     layers=layers, runs=(Run(0), Run(1)), final_norm=norm, final_norm_name="fn.",
                     head=part("linear", vocab_size=vocab, width=width, tied=True), head_name="head.")
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.weight_specs(), 9).items()}
    eng = Engine(spec, tensors, dtype="float32", max_tokens=512, max_seqs=2, poison_cache=True)
    assert not eng.use_graphs                                  # the toy part does host work: no capture

    def plain(ids):
        t = {k: v.double().cpu() for k, v in tensors.items()}
        n = len(ids)
        x = t["emb.weight"][ids]
        rms = lambda x, w: x * w / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)
        half = hd // 2
        ang = torch.arange(n, dtype=torch.float64)[:, None] * 0.3 / (torch.arange(half, dtype=torch.float64)[None] + 1)
        def rot(v):                                           # v [n, heads, hd]
            a, b = v[..., :half], v[..., half:]
            c, s_ = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
            return torch.cat([a * c - b * s_, a * s_ + b * c], -1)
        used = set()
        for p in ("a.", "b."):
            h = rms(x, t[p + "mixer_norm.weight"])
            q = rot(rms((h @ t[p + "mixer.q_proj.weight"].T).view(n, 3, hd), t[p + "mixer.q_norm.weight"]))
            k = rot(rms((h @ t[p + "mixer.k_proj.weight"].T).view(n, 3, hd), t[p + "mixer.k_norm.weight"]))
            v = (h @ t[p + "mixer.v_proj.weight"].T).view(n, 3, hd)
            o = torch.zeros(n, 3, hd, dtype=torch.float64)
            for r in range(n):
                for hh in range(3):
                    s_ = (k[:r + 1, hh] @ q[r, hh]) / math.sqrt(hd)
                    o[r, hh] = torch.softmax(s_, 0) @ v[:r + 1, hh]
            x = x + o.view(n, 3 * hd) @ t[p + "mixer.o_proj.weight"].T
            h = rms(x, t[p + "feed_forward_norm.weight"])
            if p == "a.":
                choice = (h @ t["a.feed_forward.router.weight"].T).argmax(-1)
                y = torch.zeros_like(x)
                for r in range(n):
                    e = int(choice[r])
                    used.add(e)
                    g = h[r] @ t[f"a.feed_forward.experts.{e}.gate.weight"].T
                    u_ = h[r] @ t[f"a.feed_forward.experts.{e}.up.weight"].T
                    y[r] = (g / (1 + torch.exp(-g)) * u_) @ t[f"a.feed_forward.experts.{e}.down.weight"].T
                x = x + y
            else:
                g, u_ = h @ t["b.feed_forward.gate_proj.weight"].T, h @ t["b.feed_forward.up_proj.weight"].T
                x = x + (g / (1 + torch.exp(-g)) * u_) @ t["b.feed_forward.down_proj.weight"].T
        return (rms(x, t["fn.weight"]) @ t["emb.weight"].T).numpy(), used

    ids = random_ids(4, 40, vocab)
    ref, used = plain(ids)
    assert len(used) >= 2                                      # the router does route
    s = eng.open(1)
    got = [eng.step(s, [ids[:25]], [list(range(25))]).cpu().numpy()]
    for t_ in range(25, 40):
        got.append(eng.step(s, [[ids[t_]]], [[0]]).cpu().numpy())
    eng.close(s)
    assert np.abs(np.concatenate(got) - ref).max() < 3e-5
