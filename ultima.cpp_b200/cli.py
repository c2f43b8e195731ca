"""The command line, in the manner of the reference's ``ultima`` program
(apps/ultima-cli/main.cpp:36-63 usage, :554-700 ``run``, :360-370 ``archs``): the same command
and option names where it has them.  Prompts are token ids, since the library starts at a
request's tokens: ``--prompt "1,2,3"``; several prompts are separated by ``;`` and run as a batch.

  ultima --version | --help
  ultima archs                               list known architectures and their status
  ultima archinfo <model_dir>                configuration, the tensors the model asks for, and whether
                                             the folder's files hold them (names, shapes, types)
  ultima scan <dir>                          every model folder below <dir>: runnable or why not
  ultima inspect <model_dir|file> [filter]   what the safetensors files hold: name, type, shape
  ultima random <model_dir> --config C.json [--seed N] [--dtype bfloat16|float32]
                                             write config.json and model.safetensors
  ultima run <model_dir> [--prompt IDS] [--n-predict N] [--n-ctx N] [--temp X] [--seed N]
             [--show-tokens] [--dtype bfloat16|float32] [--top-k K] [--top-p P] [--min-p P]
             [--repeat-penalty R] [--repeat-last-n N] [--stop-ids a,b] [--n-threads N]
  ultima replay ...                          same as bin/trace_run
  ultima bench ...                           same as bench.py (throughput at Qwen3-8B layer sizes)
"""
from __future__ import annotations

import json
import sys

USAGE = __doc__


def _ids(text: str) -> list:
    return [[int(x) for x in part.replace(",", " ").split()] for part in text.split(";") if part.strip()]


def cmd_archs() -> int:
    from .config import known_architectures
    from . import arch  # noqa: F401
    for e in known_architectures():
        print(f"{e.name:24s} {e.model_type:12s} {'supported' if e.supported else 'unsupported':12s} {e.notes}")
    return 0


def cmd_archinfo(argv) -> int:
    if not argv:
        print("ultima archinfo: missing model folder", file=sys.stderr)
        return 2
    from . import config_from_dir, model_spec_for
    cfg = config_from_dir(argv[0])
    print(json.dumps(cfg.to_dict(), indent=1))
    spec = model_spec_for(cfg)
    total = 0
    for s in spec.weight_specs():
        n = 1
        for d in s.shape:
            n *= d
        total += n
        print(f"{s.name:56s} {list(s.shape)}")
    print(f"{total} parameters; runs: {[r.layer for r in spec.runs]}")
    # do the folder's files hold these tensors?  (headers only; the reference's archinfo resolves
    # every tensor slot the same way, apps/ultima-cli/main.cpp:378-459)
    import os
    from .weights import WeightError, check_weights
    if os.path.isfile(os.path.join(argv[0], "model.safetensors")) or \
            os.path.isfile(os.path.join(argv[0], "model.safetensors.index.json")):
        optional = ("lm_head.weight",) if spec.head.get("tied") else ()
        try:
            found = check_weights(argv[0], spec.weight_specs(), optional)
            kinds = sorted({dt for dt, _ in found.values()})
            print(f"weights: all {len(found)} tensors present with the right shapes (stored as {', '.join(kinds)})")
        except WeightError as e:
            print(str(e))
            return 1
    else:
        print("weights: no model.safetensors in this folder")
    return 0


def _runnable(model_dir: str):
    """(True, summary) or (False, reason) for one folder with a config.json."""
    from . import ConfigError, config_from_dir, model_spec_for
    from .weights import SafetensorsError, WeightError, check_weights
    try:
        cfg = config_from_dir(model_dir)
        spec = model_spec_for(cfg)
        optional = ("lm_head.weight",) if spec.head.get("tied") else ()
        found = check_weights(model_dir, spec.weight_specs(), optional)
    except (ConfigError, WeightError, SafetensorsError, OSError, ValueError) as e:
        return False, str(e).splitlines()[0] if str(e) else type(e).__name__
    n = 0
    for _, shape in found.values():
        k = 1
        for d in shape:
            k *= d
        n += k
    return True, f"{type(cfg).__name__.replace('Config', '')}, {len(spec.layers)} layers, {n / 1e6:.1f} M parameters"


def cmd_scan(argv) -> int:
    """Every folder below the given one that holds a config.json: runnable by this library, or the
    first line of why not (the reference's ``scan`` reports the same for a folder of GGUF files,
    apps/ultima-cli/main.cpp:466-550)."""
    import os
    if not argv:
        print("ultima scan: missing folder", file=sys.stderr)
        return 2
    hits = 0
    for root, dirs, files in os.walk(argv[0]):
        dirs.sort()
        if "config.json" in files:
            hits += 1
            ok, what = _runnable(root)
            print(f"{'runnable ' if ok else 'NOT runnable'}  {root}: {what}")
    if not hits:
        print(f"no model folder (config.json) below '{argv[0]}'")
    return 0


def cmd_inspect(argv) -> int:
    """Names, types and shapes in a model folder's safetensors files, optionally only names that
    contain ``filter`` (the reference's ``--inspect <model> [filter]`` dumps its file's metadata
    and tensor table, apps/ultima-cli/main.cpp:154-244)."""
    import os
    from .weights import read_safetensors_header
    from .weights.loader import _shard_files
    if not argv:
        print("ultima inspect: missing model folder or file", file=sys.stderr)
        return 2
    paths = [argv[0]] if os.path.isfile(argv[0]) else _shard_files(argv[0])
    needle = argv[1] if len(argv) > 1 else ""
    shown = total = 0
    for path in paths:
        header, start, size = read_safetensors_header(path)
        print(f"{path}: {len(header)} tensors, header {start} bytes, file {size} bytes")
        for name in sorted(header, key=lambda n: header[n]["data_offsets"][0]):
            total += 1
            if needle and needle not in name:
                continue
            e = header[name]
            shown += 1
            print(f"  {name:56s} {e['dtype']:5s} {list(e['shape'])}")
    print(f"{shown} of {total} tensors shown")
    return 0


def cmd_random(argv) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="ultima random")
    ap.add_argument("model_dir")
    ap.add_argument("--config", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default=None, choices=["bfloat16", "float32"])
    a = ap.parse_args(argv)
    from . import config_from_dict, write_random_model
    with open(a.config) as f:
        cfg = config_from_dict(json.load(f))
    write_random_model(a.model_dir, cfg, a.seed, a.dtype)
    print(a.model_dir)
    return 0


def cmd_run(argv) -> int:
    if not argv:
        print("ultima run: missing model folder", file=sys.stderr)
        return 2
    model_dir = argv[0]
    opt = {"prompt": "1,2,3", "n_predict": 48, "n_ctx": 512, "temp": 0.0, "seed": 0, "show_tokens": False,
           "dtype": "bfloat16", "top_k": 0, "top_p": 1.0, "min_p": 0.0, "repeat_penalty": 1.0,
           "repeat_last_n": 0, "stop_ids": None, "n_threads": 0}
    conv = {"prompt": str, "n_predict": int, "n_ctx": int, "temp": float, "seed": int, "dtype": str,
            "top_k": int, "top_p": float, "min_p": float, "repeat_penalty": float, "repeat_last_n": int,
            "stop_ids": str, "n_threads": int}
    i = 1
    while i < len(argv):
        a = argv[i]
        key = a[2:].replace("-", "_") if a.startswith("--") else None
        if key == "show_tokens":
            opt[key] = True
        elif key in conv:
            if i + 1 >= len(argv):
                print(f"ultima run: {a} requires a value", file=sys.stderr)
                return 2
            i += 1
            opt[key] = conv[key](argv[i])
        else:
            print(f"ultima run: unknown flag '{a}'", file=sys.stderr)
            return 2
        i += 1
    from .engine.generate import LLM
    from .sampling import SamplingParams
    prompts = _ids(opt["prompt"])
    if opt["show_tokens"]:
        for p in prompts:
            print("prompt tokens:", " ".join(map(str, p)))
    for p in prompts:
        if len(p) + opt["n_predict"] > opt["n_ctx"]:
            print(f"ultima run: prompt ({len(p)}) + n-predict ({opt['n_predict']}) exceeds n-ctx "
                  f"({opt['n_ctx']})", file=sys.stderr)
            return 1
    llm = LLM(model_dir, dtype=opt["dtype"], n_ctx=opt["n_ctx"], max_batch=max(1, len(prompts)))
    mem = llm.engine.memory_report()
    print(f"[weights {mem['weights'] / 2**20:.1f} MiB | cache {mem['cache'] / 2**20:.1f} MiB for {mem['cache_positions']} "
          f"positions in {mem['slots']} slots | scratch {mem['scratch'] / 2**20:.1f} MiB]", file=sys.stderr)
    sp = SamplingParams(temperature=opt["temp"], top_k=opt["top_k"], top_p=opt["top_p"], min_p=opt["min_p"],
                        rep_penalty=opt["repeat_penalty"], repeat_last_n=opt["repeat_last_n"])
    stop = None if opt["stop_ids"] is None else [int(x) for x in opt["stop_ids"].replace(",", " ").split()]
    outs = llm.generate(prompts, n_predict=opt["n_predict"], seed=opt["seed"], stop_token_ids=stop, sampling=sp)
    for g in outs:
        print(" ".join(map(str, g.tokens)))
    st = llm.last_stats
    pre = st.prompt_tokens / st.prefill_s if st.prefill_s > 0 else 0.0
    dec = (st.generated_tokens - len(prompts)) / st.decode_s if st.decode_s > 0 else 0.0
    print(f"[{st.prompt_tokens} prompt tok in {st.prefill_s * 1e3:.1f} ms ({pre:.1f} tok/s) | "
          f"{st.generated_tokens} gen tok in {st.decode_s * 1e3:.1f} ms ({dec:.1f} tok/s)]", file=sys.stderr)
    if st.device_step_ms:
        steps = sorted(st.device_step_ms)
        print(f"[on the device: prompt step {st.device_prefill_ms:.2f} ms | {len(steps)} decode steps, "
              f"median {steps[len(steps) // 2]:.3f} ms, longest {steps[-1]:.3f} ms]", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("--help", "-h", "help"):
        print(USAGE)
        return 0
    if argv[0] == "--version":
        from . import __version__
        print(f"ultima_b200 {__version__}")
        return 0
    cmd, rest = argv[0], argv[1:]
    try:
        if cmd == "archs":
            return cmd_archs()
        if cmd == "archinfo":
            return cmd_archinfo(rest)
        if cmd == "scan":
            return cmd_scan(rest)
        if cmd in ("inspect", "--inspect"):
            return cmd_inspect(rest)
        if cmd == "random":
            return cmd_random(rest)
        if cmd == "run":
            return cmd_run(rest)
        if cmd == "replay":
            from .engine.trace import main as replay_main
            return replay_main(rest)
        if cmd == "bench":
            import os
            import runpy
            root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
            sys.argv = ["bench.py"] + rest
            runpy.run_path(os.path.join(root, "bench.py"), run_name="__main__")
            return 0
    except (ValueError, RuntimeError, OSError) as e:
        print(f"ultima {cmd}: {e}", file=sys.stderr)
        return 1
    print(f"ultima: unknown command '{cmd}'\n", file=sys.stderr)
    print(USAGE, file=sys.stderr)
    return 2
