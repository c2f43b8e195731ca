"""A whole architecture that exists only in this file, taken through everything a real one goes through
without a change to the package: a typed configuration with keys of its own, a function from the
configuration to the model as data, an entry in the registry, a model folder written from a seed
(config.json and model.safetensors under the architecture's own tensor names), the loader, the engine,
the generation loop; every logit against a plain implementation written here from the plain parts.

The architecture is made up for the test ("ToyTwin"): no per-head norm of q and k, a rotation of
interleaved pairs over the first half of every head only, an attention scale of its own, a window on
some layers, its first layer run a second time at the end of the stack (weights shared, a cache of its
own), tied or untied output."""
import dataclasses
import math
import os

import numpy as np
import pytest

from conftest import close_enough

pytestmark = pytest.mark.gpu


@dataclasses.dataclass(frozen=True)
class ToyTwinConfig:
    vocab: int
    width: int
    depth: int
    heads: int
    kv_heads: int
    head_size: int
    inner: int
    eps: float
    theta: float
    score_scale: float
    window: int
    window_layers: tuple
    tied: bool
    max_position_embeddings: int
    torch_dtype: str = "bfloat16"
    architecture: str = "ToyTwinForCausalLM"

    @classmethod
    def from_dict(cls, d):
        from ultima_b200.config.base import ConfigError
        for key in ("vocab", "width", "depth", "heads", "kv_heads", "head_size", "inner", "max_position_embeddings"):
            if not isinstance(d.get(key), int) or d[key] < 1:
                raise ConfigError(f"config.json: '{key}' must be a positive integer")
        return cls(vocab=d["vocab"], width=d["width"], depth=d["depth"], heads=d["heads"], kv_heads=d["kv_heads"],
                   head_size=d["head_size"], inner=d["inner"], eps=float(d["eps"]), theta=float(d["theta"]),
                   score_scale=float(d["score_scale"]), window=int(d.get("window", 0)),
                   window_layers=tuple(d.get("window_layers", ())), tied=bool(d.get("tied", False)),
                   max_position_embeddings=d["max_position_embeddings"], torch_dtype=d.get("torch_dtype", "bfloat16"))

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["window_layers"] = list(self.window_layers)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "toy_twin"
        return d


def _build_spec(cfg: ToyTwinConfig, max_positions=None):
    from ultima_b200.parts.base import ModelSpec, Run, layer, part
    max_pos = int(max_positions or cfg.max_position_embeddings)
    position = part("rotary_interleaved", head_dim=cfg.head_size, theta=cfg.theta, max_positions=max_pos,
                    rotary_dim=cfg.head_size // 2)
    norm = part("rms", width=cfg.width, eps=cfg.eps)
    names = (("mixer", "mix."), ("feed_forward", "ffn."), ("mixer_norm", "n1."), ("feed_forward_norm", "n2."))
    layers = []
    for i in range(cfg.depth):
        mixer = part("attention", width=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_size,
                     qk_norm=False, eps=cfg.eps, position=position, scale=cfg.score_scale,
                     window=cfg.window if i in cfg.window_layers else None)
        layers.append(layer(part("pre_norm"), prefix=f"blocks.{i}.", names=names, mixer=mixer,
                            feed_forward=part("gated_silu", width=cfg.width, inner=cfg.inner),
                            mixer_norm=norm, feed_forward_norm=norm))
    return ModelSpec(width=cfg.width, vocab_size=cfg.vocab, max_positions=max_pos,
                     embedding=part("token_table", vocab_size=cfg.vocab, width=cfg.width), embedding_name="emb.",
                     layers=tuple(layers), runs=tuple(Run(i) for i in range(cfg.depth)) + (Run(0),),
                     final_norm=norm, final_norm_name="out_norm.",
                     head=part("linear", vocab_size=cfg.vocab, width=cfg.width, tied=cfg.tied), head_name="out.")


def _register():
    from ultima_b200.config.base import ArchitectureEntry, register_architecture
    register_architecture(ArchitectureEntry("ToyTwinForCausalLM", "toy_twin", True, "made up for a test",
                                            ToyTwinConfig, _build_spec), replace=True)


CONFIGS = {
    "small": dict(architectures=["ToyTwinForCausalLM"], vocab=211, width=96, depth=2, heads=6, kv_heads=2, head_size=32,
                  inner=160, eps=3e-6, theta=5000.0, score_scale=0.2, window=20, window_layers=[1], tied=True,
                  max_position_embeddings=256),
    "tc": dict(architectures=["ToyTwinForCausalLM"], vocab=307, width=192, depth=3, heads=4, kv_heads=1, head_size=64,
               inner=320, eps=1e-5, theta=20000.0, score_scale=0.11, window=0, window_layers=[], tied=False,
               max_position_embeddings=256),
}


# ---- the plain implementation of this architecture, from the plain parts ------------------------------
def _rotate_interleaved_part(x, positions, theta, rotary_dim):
    """Pairs (x[2j], x[2j + 1]) of the first ``rotary_dim`` columns by pos * theta^(-2j / rotary_dim); the
    other columns pass through (the reference's rotation with a rotated sub-range, src/kernels/rope.cpp:27-50,
    with the interleaved pairing of its registry, include/ultima/model/arch_registry.hpp:32-38)."""
    half = rotary_dim // 2
    j = np.arange(half, dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] / np.power(float(theta), 2.0 * j / rotary_dim)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
    out[..., 0:rotary_dim:2] = a * c - b * s
    out[..., 1:rotary_dim:2] = a * s + b * c
    return out


def _plain_forward(cfg, w, ids):
    import plain_qwen3 as P
    T = len(ids)
    pos = np.arange(T)
    nh, nkv, d = cfg["heads"], cfg["kv_heads"], cfg["head_size"]
    x = P.embed(w["emb.weight"], ids)
    for i in list(range(cfg["depth"])) + [0]:
        pre = f"blocks.{i}."
        h = P.rmsnorm(x, w[pre + "n1.weight"], cfg["eps"])
        q = P.linear(h, w[pre + "mix.q_proj.weight"]).reshape(T, nh, d)
        k = P.linear(h, w[pre + "mix.k_proj.weight"]).reshape(T, nkv, d)
        v = P.linear(h, w[pre + "mix.v_proj.weight"]).reshape(T, nkv, d)
        q = _rotate_interleaved_part(q, pos, cfg["theta"], d // 2)
        k = _rotate_interleaved_part(k, pos, cfg["theta"], d // 2)
        # the plain attention scales by 1 / sqrt(d): this architecture's own scale goes onto q
        q = q * (cfg["score_scale"] * math.sqrt(d))
        window = cfg["window"] if i in cfg["window_layers"] else None
        o = P.attention(q, k, v, pos, window).reshape(T, nh * d)
        x = x + P.linear(o, w[pre + "mix.o_proj.weight"])
        h = P.rmsnorm(x, w[pre + "n2.weight"], cfg["eps"])
        x = x + P.linear(P.swiglu(P.linear(h, w[pre + "ffn.gate_proj.weight"]), P.linear(h, w[pre + "ffn.up_proj.weight"])),
                         w[pre + "ffn.down_proj.weight"])
    x = P.rmsnorm(x, w["out_norm.weight"], cfg["eps"])
    return P.linear(x, w["emb.weight"] if cfg["tied"] else w["out.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "tc"])
def test_an_architecture_of_the_tests_own_from_folder_to_tokens(tmp_path, name, dtype):
    import plain_qwen3 as P
    import ultima_b200 as u
    from ultima_b200.config.base import known_architectures
    from ultima_b200.engine import Engine
    _register()
    assert any(e.name == "ToyTwinForCausalLM" and e.supported for e in known_architectures())
    cfg = u.config_from_dict(CONFIGS[name])
    assert isinstance(cfg, ToyTwinConfig) and cfg.window_layers == tuple(CONFIGS[name]["window_layers"])
    model_dir = str(tmp_path / name)
    u.write_random_model(model_dir, cfg, seed=11, dtype="bfloat16")
    assert u.config_from_dir(model_dir) == dataclasses.replace(cfg, torch_dtype="bfloat16")
    pcfg, w = P.read_folder(model_dir)
    assert "blocks.0.mix.q_proj.weight" in w and ("out.weight" in w) == (not pcfg["tied"])

    eng = Engine.from_dir(model_dir, dtype=dtype, max_tokens=512, max_seqs=3, poison_cache=True)
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, pcfg["vocab"], size=n).tolist() for n in (97, 40, 131)]
    cut = [97 - 12, 40 - 12, 131 - 12]
    slots = eng.open(3)
    got = [dict() for _ in seqs]
    out = eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
    o = 0
    for i, c in enumerate(cut):
        for pl in range(c):
            got[i][pl] = out[o]
            o += 1
    for t in range(12):                                    # the last twelve tokens one by one, as a batch
        out = eng.step(slots, [[s[c + t]] for s, c in zip(seqs, cut)]).cpu().numpy()
        for i, c in enumerate(cut):
            got[i][c + t] = out[i]
    eng.close(slots)
    eng.check_errors()
    n_runs = pcfg["depth"] + 1
    for i, ids in enumerate(seqs):
        ref = _plain_forward(pcfg, w, ids)
        g = np.stack([got[i][pl] for pl in range(len(ids))])
        err, bound = close_enough(g, ref, dtype, n_runs)
        assert err <= bound, (name, dtype, i, err, bound)

    # and through the generation loop: greedy tokens as the plain implementation picks them (32-bit only:
    # where two logits are close bfloat16 may pick the other)
    if dtype == "float32":
        llm = u.LLM(model_dir, dtype="float32", n_ctx=128, max_batch=2)
        prompts = [seqs[0][:9], seqs[1][:4]]
        outs = llm.generate(prompts, n_predict=6, temp=0.0)
        for p, g in zip(prompts, outs):
            ids = list(p)
            for _ in range(6):
                ids.append(P.argmax_first(_plain_forward(pcfg, w, ids)[-1]))
            assert g.tokens == ids[len(p):], (name, g.tokens, ids[len(p):])


def test_the_toy_architecture_is_listed_and_refuses_a_bad_configuration():
    import ultima_b200 as u
    from ultima_b200.config.base import ConfigError
    _register()
    bad = dict(CONFIGS["small"])
    bad["heads"] = 0
    with pytest.raises(ConfigError):
        u.config_from_dict(bad)
    spec = u.model_spec_for(u.config_from_dict(CONFIGS["small"]))
    names = {s.name for s in spec.weight_specs()}
    assert "blocks.1.ffn.down_proj.weight" in names and "out.weight" not in names      # tied: no output matrix
    assert [r.layer for r in spec.runs] == [0, 1, 0]
    assert os.path.basename(__file__).startswith("test_")


def test_the_command_line_programs_take_an_architecture_from_outside_the_package(tmp_path):
    """``bin/trace_run`` and ``bin/ultima`` are processes of their own: a module named in ULTIMA_ARCH_MODULES
    enters its architecture into their registry.  The module here imports this test file's definitions."""
    import json
    import subprocess
    import sys
    import plain_qwen3 as P
    import ultima_b200 as u
    from conftest import ROOT
    _register()
    cfg = u.config_from_dict(CONFIGS["tc"])
    model_dir = str(tmp_path / "tc")
    u.write_random_model(model_dir, cfg, seed=12, dtype="bfloat16")
    plug = tmp_path / "plug"
    plug.mkdir()
    (plug / "toy_twin_arch.py").write_text("import test_toy_architecture_gpu as t\nt._register()\n")
    env = dict(os.environ)
    env["ULTIMA_ARCH_MODULES"] = "toy_twin_arch"
    env["PYTHONPATH"] = os.pathsep.join([str(plug), os.path.dirname(os.path.abspath(__file__)), env.get("PYTHONPATH", "")])
    listed = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ultima"), "archs"], env=env, capture_output=True,
                            text=True, timeout=300)
    assert listed.returncode == 0 and "ToyTwinForCausalLM" in listed.stdout, listed.stderr[-1500:]
    pcfg, w = P.read_folder(model_dir)
    rng = np.random.default_rng(8)
    a, b = rng.integers(0, pcfg["vocab"], size=70).tolist(), rng.integers(0, pcfg["vocab"], size=9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + t]], "want": [0]}],
                      "end": ["a", "b"] if t == 3 else []})
    out_dir = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps),
                       env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ra, rb = _plain_forward(pcfg, w, a), _plain_forward(pcfg, w, b)
    first = np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(3, pcfg["vocab"])
    want = [ra[0], ra[65], rb[4]]
    for t in range(4):
        rows = np.fromfile(os.path.join(out_dir, f"{t + 1}.f32"), dtype="<f4").reshape(2, pcfg["vocab"])
        first = np.concatenate([first, rows])
        want += [ra[66 + t], rb[5 + t]]
    err, bound = close_enough(first, np.stack(want), "float32", pcfg["depth"] + 1)
    assert err <= bound, (err, bound)
