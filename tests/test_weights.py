"""Weights: the safetensors container, loading by name, the one error, random folders (no GPU)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
import ultima_b200 as u
from ultima_b200.weights import (WeightError, SafetensorsError, load_weights, open_safetensors,
                                 write_safetensors, storage_dtype, random_tensors)


def _folder(tmp_path, d=TINY_B, dtype="bfloat16", seed=3):
    cfg = u.config_from_dict(d)
    return cfg, u.write_random_model(str(tmp_path / "m"), cfg, seed, dtype)


def test_random_folder_reads_back(tmp_path):
    cfg, d = _folder(tmp_path)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert u.config_from_dir(d) == cfg
    spec = u.model_spec_for(cfg)
    t = load_weights(d, spec.weight_specs(), torch.bfloat16)
    assert t["model.layers.2.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert t["model.layers.2.mlp.down_proj.weight"].shape == (96, 320)
    assert t["model.norm.weight"].dtype == torch.float32           # vectors are widened
    w = t["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = t["model.layers.1.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.03
    t32 = load_weights(d, spec.weight_specs(), torch.float32)
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["lm_head.weight"], t["lm_head.weight"].float())


def test_same_seed_same_weights_other_seed_other(tmp_path):
    cfg = u.config_from_dict(TINY_A)
    specs = u.model_spec_for(cfg).weight_specs()
    a, b, c = random_tensors(specs, 5), random_tensors(specs, 5), random_tensors(specs, 6)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])


def test_storage_types():
    assert storage_dtype("BF16", torch.bfloat16, "matrix") == torch.bfloat16
    assert storage_dtype("F32", torch.bfloat16, "matrix") == torch.float32      # 32-bit stays
    assert storage_dtype("F16", torch.bfloat16, "matrix") == torch.bfloat16
    assert storage_dtype("BF16", torch.float32, "matrix") == torch.float32
    assert storage_dtype("I64", torch.bfloat16, "table") == torch.int32
    assert storage_dtype("BF16", torch.bfloat16, "vector") == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, d = _folder(tmp_path, dtype="float32")
    f = open_safetensors(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    del tensors["model.layers.1.self_attn.k_norm.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    tensors["model.layers.2.mlp.up_proj.weight"] = torch.zeros(320, 95)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as ei:
        load_weights(d, u.model_spec_for(cfg).weight_specs(), torch.float32)
    e = ei.value
    assert sorted(e.missing) == ["model.layers.1.self_attn.k_norm.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert e.wrong_shape == [("model.layers.2.mlp.up_proj.weight", (320, 96), (320, 95))]
    msg = str(e)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "expected [320, 96], got [320, 95]"):
        assert piece in msg


def test_tied_model_may_carry_a_head_and_untied_must(tmp_path):
    cfg = u.config_from_dict(TINY_A)
    d = u.write_random_model(str(tmp_path / "t"), cfg, 1, "float32")
    spec = u.model_spec_for(cfg)
    f = open_safetensors(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(d, spec.weight_specs(), torch.float32)
    load_weights(d, spec.weight_specs(), torch.float32, optional=("lm_head.weight",))


def test_container_faults(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
                          "b": torch.ones(4, dtype=torch.bfloat16), "c": torch.arange(3, dtype=torch.int64)})
    f = open_safetensors(p)
    assert f.info("a") == ("F32", (2, 3)) and f.info("b") == ("BF16", (4,))
    assert torch.equal(f.tensor("a"), torch.arange(6, dtype=torch.float32).reshape(2, 3))
    assert f.tensor("b").dtype == torch.bfloat16 and f.tensor("c").tolist() == [0, 1, 2]
    f.close()
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-5])                                   # truncated data
    with pytest.raises(SafetensorsError, match="outside the data section"):
        open_safetensors(p)
    open(p, "wb").write(struct.pack("<Q", 10) + b"not json!!" + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="not JSON"):
        open_safetensors(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        open_safetensors(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlap"):
        open_safetensors(p)


def test_reads_files_of_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    p = str(tmp_path / "y.safetensors")
    a = torch.randn(5, 7).to(torch.bfloat16)
    st.save_file({"w": a}, p)
    f = open_safetensors(p)
    assert torch.equal(f.tensor("w"), a)
    f.close()
    q = str(tmp_path / "z.safetensors")
    write_safetensors(q, {"w": a})
    assert torch.equal(st.load_file(q)["w"], a)


def test_sharded_folder_is_read_through_its_index(tmp_path):
    cfg, d = _folder(tmp_path, d=TINY_A, dtype="float32")
    f = open_safetensors(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[:len(names) // 2],
             "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    weight_map = {}
    for fn, ns in parts.items():
        write_safetensors(os.path.join(d, fn), {n: tensors[n] for n in ns})
        weight_map.update({n: fn for n in ns})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"metadata": {}, "weight_map": weight_map}, fh)
    got = load_weights(d, u.model_spec_for(cfg).weight_specs(), torch.float32)
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_command_line_reports_on_folders_without_a_gpu(tmp_path, capsys):
    """archinfo, scan and inspect read configuration and file headers only."""
    import copy
    import json as _json
    from conftest import TINY_A, TINY_B
    from ultima_b200.cli import main
    good, bad = tmp_path / "zoo" / "good", tmp_path / "zoo" / "bad"
    u.write_random_model(str(good), u.config_from_dict(copy.deepcopy(TINY_A)), seed=1)
    u.write_random_model(str(bad), u.config_from_dict(copy.deepcopy(TINY_B)), seed=2)
    cfg = _json.loads((bad / "config.json").read_text())
    cfg["intermediate_size"] += 64                       # the files no longer fit the configuration
    (bad / "config.json").write_text(_json.dumps(cfg))
    assert main(["archinfo", str(good)]) == 0
    out = capsys.readouterr().out
    assert "model.layers.0.self_attn.q_proj.weight" in out and "all" in out and "tensors present" in out
    assert main(["archinfo", str(bad)]) == 1
    assert "wrong shape" in capsys.readouterr().out
    assert main(["scan", str(tmp_path / "zoo")]) == 0
    out = capsys.readouterr().out
    lines = [l for l in out.splitlines() if l.strip()]
    assert len(lines) == 2
    assert any(l.startswith("runnable") and "good" in l for l in lines)
    assert any(l.startswith("NOT runnable") and "bad" in l for l in lines)
    assert main(["inspect", str(good), "q_norm"]) == 0
    out = capsys.readouterr().out
    assert "q_norm.weight" in out and "k_norm" not in out and "tensors shown" in out
