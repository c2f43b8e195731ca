"""Trace replay: given token ids go through the engine step by step and the logits are
written out.  Nothing is sampled.  It drives the same model, step function, cache and
kernels as generation; it has no forward pass of its own.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted
places in the order of the entries and of ``want`` (little-endian float32, [wanted, vocab]).
After every step a line ``done <step>`` is printed.

The reference has nothing of this kind; its nearest tools are the per-layer checksum lines
of ULTIMA_TRACE (src/model/qwen_block.cpp:29-42) and benchmarks/check_taps.cpp.
"""
from __future__ import annotations

import json
import os
import sys


def replay(engine, lines, out_dir: str, say=None) -> int:
    """Feed ``lines`` (an iterable of JSON strings) through ``engine``; returns the number of
    steps run."""
    os.makedirs(out_dir, exist_ok=True)
    slot_of: dict = {}
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        slots, tokens, want = [], [], []
        for e in entries:
            rid = e["id"]
            if rid not in slot_of:
                slot_of[rid] = engine.open(1)[0]
            slots.append(slot_of[rid])
            tokens.append([int(t) for t in e["tokens"]])
            want.append([int(p) for p in e.get("want", [])])
        if entries:
            logits = engine.step(slots, tokens, want)
            engine.check_errors()
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            if rid in slot_of:
                engine.close([slot_of.pop(rid)])
        n += 1
        if say is not None:
            say(f"done {step}")
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the "
                                 "engine step by step and write the logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--max-step-tokens", type=int, default=4096)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    def say(msg):
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    print(f"[trace_run] loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    from .engine import Engine
    engine = Engine.from_dir(args.model, dtype=args.dtype, max_tokens=args.max_tokens,
                             max_step_tokens=args.max_step_tokens, device=args.device, with_sampler=False)
    engine.warm_up()
    print("[trace_run] ready", file=sys.stderr, flush=True)
    replay(engine, sys.stdin, args.out, say)
    return 0
