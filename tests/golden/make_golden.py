#!/usr/bin/env python3
"""Makes tests/golden/tiny_{A,B,C}.npz: the logits of the reference's own model code
(tattooinmtl/Ultima.cpp, compiled unchanged for the CPU) on three tiny Qwen3 models (C has a
sliding window on two of its three layers).

    python tests/golden/make_golden.py /path/to/Ultima.cpp [build_dir]

The reference's CMake build fetches its dependencies from the network and its file loader is
for Windows only, so this script compiles the translation units of the model path directly with
g++ (C++23, AVX2), with two small stand-ins on the include path: ``nonstd/expected.hpp``
forwarding to ``<expected>`` and the header-only ``fmt`` that ships inside the torch wheel.
``harness.cpp`` (beside this file) serves the model through the reference's abstract
``LoadedModel``.  Weights come from ``golden_weights.py``.  Stored: the logits of token-by-token
decode at the kept positions, the logits of a whole-prompt prefill (last position), and the
largest difference between the two (the reference gives exactly 0).
"""
import glob
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import golden_weights as G  # noqa: E402

MODEL_SRCS = ["dtype", "tensor_info", "metadata_store", "loaded_model", "arch_registry", "qwen_config",
              "qwen_tensor_slots", "weight_dispatch", "qwen_block", "qwen_model", "hadamard"]


def build(ref: str, bdir: str) -> str:
    inc = os.path.join(bdir, "inc")
    os.makedirs(os.path.join(inc, "nonstd"), exist_ok=True)
    os.makedirs(os.path.join(bdir, "obj"), exist_ok=True)
    import torch
    fmt = os.path.join(os.path.dirname(torch.__file__), "include", "fmt")
    if not os.path.exists(os.path.join(inc, "fmt")):
        os.symlink(fmt, os.path.join(inc, "fmt"))
    with open(os.path.join(inc, "nonstd", "expected.hpp"), "w") as f:
        f.write("#pragma once\n#include <expected>\nnamespace nonstd { using std::expected; using std::unexpected; }\n")
    srcs = ["src/core/error.cpp", "src/runtime/thread_pool.cpp", "src/kv_cache/kv_cache.cpp",
            "src/kv_cache/recurrent_state.cpp", "src/sampler/sampler.cpp"]
    srcs += sorted(os.path.relpath(p, ref) for p in glob.glob(os.path.join(ref, "src/kernels/*.cpp")))
    srcs += [f"src/model/{s}.cpp" for s in MODEL_SRCS]
    flags = ["-std=c++23", "-O2", "-mavx2", "-mfma", "-DFMT_HEADER_ONLY", "-include", "immintrin.h",
             "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "src/model"), "-isystem", inc]
    procs = []
    for s in srcs:
        obj = os.path.join(bdir, "obj", s.replace("/", "_") + ".o")
        if not os.path.exists(obj):
            procs.append(subprocess.Popen(["g++"] + flags + ["-c", os.path.join(ref, s), "-o", obj]))
        if len(procs) >= 8:
            for p in procs:
                assert p.wait() == 0
            procs = []
    for p in procs:
        assert p.wait() == 0
    exe = os.path.join(bdir, "harness")
    objs = sorted(glob.glob(os.path.join(bdir, "obj", "*.o")))
    subprocess.check_call(["g++"] + flags + [os.path.join(HERE, "harness.cpp")] + objs + ["-lpthread", "-o", exe])
    return exe


def run(exe: str, name: str, bdir: str):
    cfg, toks = G.CONFIGS[name], G.PROMPTS[name]
    w = G.weights(cfg)
    inp, out = os.path.join(bdir, f"{name}.in"), os.path.join(bdir, f"{name}.out")
    with open(inp, "wb") as f:
        f.write(struct.pack("<11i", cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"],
                            cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                            cfg["vocab_size"], cfg["max_position_embeddings"], int(cfg["tie_word_embeddings"]),
                            len(toks), int(cfg.get("sliding_window") or 0)))
        types = cfg.get("layer_types") or ["full_attention"] * cfg["num_hidden_layers"]
        f.write(struct.pack(f"<{len(types)}i", *[int(t == "sliding_attention") for t in types]))
        f.write(struct.pack("<2f", cfg["rms_norm_eps"], cfg["rope_theta"]))
        f.write(np.asarray(toks, dtype="<i4").tobytes())
        for n, _, _ in G.tensor_list(cfg):
            f.write(w[n].astype("<f4").tobytes())
    subprocess.check_call([exe, inp, out])
    V = cfg["vocab_size"]
    a = np.fromfile(out, dtype="<f4").reshape(len(toks) + 1, V)
    decode, prefill_last = a[:-1], a[-1]
    diff = float(np.abs(decode[-1] - prefill_last).max())
    np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), positions=np.asarray(G.KEPT[name]),
                        decode_logits=decode[G.KEPT[name]], prefill_last_logits=prefill_last,
                        prefill_vs_decode_max_abs=np.float64(diff))
    print(name, "max |logit|", float(np.abs(decode).max()), "prefill vs decode", diff)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of tattooinmtl/Ultima.cpp> [build folder]")
    ref = sys.argv[1]
    bdir = sys.argv[2] if len(sys.argv) > 2 else os.path.join(tempfile.gettempdir(), "ultima_golden_build")
    exe = build(ref, bdir)
    for name in ("A", "B", "C"):
        run(exe, name, bdir)
