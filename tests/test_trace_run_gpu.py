"""bin/trace_run as a user calls it: a child process, steps on standard input, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, random_ids, close_enough

pytestmark = pytest.mark.gpu


def _run(model_dir, dtype, out_dir, steps, max_tokens):
    inp = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
                        "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                       input=inp, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    return p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_batches_of_unequal_lengths(model_dirs, plain_models, tmp_path, dtype):
    import plain_qwen3 as P
    name = "C"
    cfg, w = plain_models(name, "bfloat16")
    V = cfg["vocab_size"]
    reqs = {"a": random_ids(1, 40, V), "b": random_ids(2, 7, V), "c": random_ids(3, 70, V), "d": random_ids(4, 5, V)}
    prompt = {"a": 30, "b": 4, "c": 66, "d": 1}
    steps, n = [], 0
    for batch in (["a", "b"], ["c", "d"]):        # the second batch reuses what the first gave back
        steps.append({"step": n, "entries": [{"id": r, "tokens": reqs[r][:prompt[r]],
                                               "want": list(range(prompt[r]))} for r in batch], "end": []})
        n += 1
        t = 0
        live = list(batch)
        while live:
            going = [r for r in live if prompt[r] + t < len(reqs[r])]
            if not going:
                steps[-1]["end"] = live
                break
            ending = [r for r in going if prompt[r] + t + 1 >= len(reqs[r])] + [r for r in live if r not in going]
            steps[-1]["end"] += [r for r in live if r not in going]
            steps.append({"step": n, "entries": [{"id": r, "tokens": [reqs[r][prompt[r] + t]], "want": [0]}
                                                  for r in going], "end": []})
            n += 1
            live = going
            t += 1
    out_dir = str(tmp_path / "out")
    # 40 -> 64 and 7 -> 64: 128 positions live at most in batch one; 70 -> 128 and 5 -> 64 in batch two
    _run(model_dirs(name, "bfloat16"), dtype, out_dir, steps, max_tokens=192)
    got = {r: [] for r in reqs}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        rows = sum(len(e["want"]) for e in s["entries"])
        arr = np.fromfile(path, dtype="<f4").reshape(rows, V)
        o = 0
        for e in s["entries"]:
            got[e["id"]].append(arr[o:o + len(e["want"])])
            o += len(e["want"])
    for r, ids in reqs.items():
        g = np.concatenate(got[r])
        err, bound = close_enough(g, P.forward(cfg, w, ids), dtype, cfg["num_hidden_layers"])
        assert err <= bound, (r, err, bound)


def test_replay_writes_no_file_when_nothing_is_wanted(model_dirs, tmp_path):
    out_dir = str(tmp_path / "o2")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": [4], "want": [0]}], "end": ["x"]}]
    _run(model_dirs("A", "float32"), "float32", out_dir, steps, 64)
    assert sorted(os.listdir(out_dir)) == ["1.f32"]
    assert os.path.getsize(os.path.join(out_dir, "1.f32")) == 512 * 4
