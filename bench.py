#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output.  A step is one decode step of a batch of 8 sequences whose
prompts (2,048 random token ids each) are already in the cache; ``value`` is decoded tokens
a second, timed on the device with CUDA events around exactly K steps after W warm-up steps.
``e2e`` is the same through the Python entry point (``LLM.generate``): token ids from the host in,
sampled ids back on the host every step; on the host's clock, again exactly K steps after W
warm-up steps (the prompts and the steps right after them, which the device runs more slowly,
are outside the timed region, as they are for ``value``).  ``prefill`` times one 2,048-token prompt; ``points`` gives
decode at batch 1 and 64; ``roofline`` compares the bytes a decode step has to read (every
weight once, the cache of the live sequences) with the measured copy bandwidth.
Weights are random from a seed (there is no checkpoint offline); the step reads 15 GB of
weights, far more than the 126 MB L2, so no flush is needed between timed steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936,
                hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                rope_theta=1000000.0, max_position_embeddings=8192, tie_word_embeddings=False,
                hidden_act="silu")
PROMPT, CONTEXT, BATCH, PREFILL_TOKENS = 2048, 8192, 8, 2048

# the other two workloads the baseline names (layer sizes of Qwen3-14B and Qwen3-32B, random weights)
OTHER = {
    "14b": dict(sizes=dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40,
                           num_key_value_heads=8, head_dim=128), batch=16, prompt=("uniform", 128, 4096), decode=256),
    "32b": dict(sizes=dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                           num_key_value_heads=8, head_dim=128), batch=8, prompt=("fixed", 4096, 4096), decode=512),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v == "Active"})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def weight_bytes(cfg, dtype_bytes=2):
    """Every weight a decode step uses, once: the projections of each layer and the head (the
    embedding table is read one row a token; norm weights are counted)."""
    H, Q, KV, F, V, L = (cfg.hidden_size, cfg.q_width, cfg.kv_width, cfg.intermediate_size,
                         cfg.vocab_size, cfg.num_hidden_layers)
    mats = L * (H * (Q + 2 * KV) + Q * H + 3 * H * F) + V * H
    vecs = L * (2 * H + 2 * cfg.head_dim) + H
    return mats * dtype_bytes + vecs * 4


def kv_bytes_per_token(cfg, dtype_bytes):
    return 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * dtype_bytes


def prefill_flops(cfg, T):
    H, Q, KV, F, V, L = (cfg.hidden_size, cfg.q_width, cfg.kv_width, cfg.intermediate_size,
                         cfg.vocab_size, cfg.num_hidden_layers)
    linear = 2 * T * L * (H * (Q + 2 * KV) + Q * H + 3 * H * F)
    attn = L * 4 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) // 2)
    return linear + attn + 2 * V * H


def fill_cache(engine, slots, n_tokens):
    """Put ``n_tokens`` positions of random keys and values into each slot without running the
    model (what they hold does not change a decode step's time)."""
    for s in slots:
        engine.cache.reserve(s, n_tokens)
        engine.cache.commit(s, n_tokens)


def measured_peaks():
    """What this GPU gives a plain device-to-device copy (bytes read + bytes written a second, 4 GiB a
    buffer) and the library's bfloat16 product (8192^3, a burst of 20 and a loop of about two seconds):
    the same kind of figures as the denominators in MEASURED_PEAKS.json, for the box a run was taken on;
    and the library's product on the four shapes of a prompt layer.  Nothing of the library under test
    runs here."""
    import torch
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    n = 1 << 30
    a = torch.empty(n, dtype=torch.float32, device=dev).normal_()
    b = torch.empty_like(a)

    def timed(fn, reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for _ in range(3):
        b.copy_(a)
    copy_ms = timed(lambda: b.copy_(a), 10)
    copy_gbs = 2 * a.numel() * 4 / (copy_ms * 1e-3) / 1e9
    del a, b
    m = 8192
    x = torch.randn(m, m, device=dev, dtype=torch.bfloat16)
    y = torch.randn(m, m, device=dev, dtype=torch.bfloat16)
    out = torch.empty(m, m, device=dev, dtype=torch.bfloat16)
    for _ in range(5):
        torch.matmul(x, y, out=out)
    burst_ms = timed(lambda: torch.matmul(x, y, out=out), 20)
    flop = 2.0 * m * m * m
    reps = max(20, int(2000 / burst_ms))
    clocks = ClockSampler()
    clocks.start()
    loop_ms = timed(lambda: torch.matmul(x, y, out=out), reps)
    clk = clocks.stop()
    # the library's product on the four shapes of a 2,048-token prompt's layer (weights rotated so that they
    # come from memory as in a model): what these shapes allow, against the 8192^3 figure the fractions use
    shapes = {}
    c = QWEN3_8B
    q, kv, h, f = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"], c["hidden_size"], c["intermediate_size"]
    for name, n, k in (("qkv", q + 2 * kv, h), ("output", h, q), ("gate_up", 2 * f, h), ("down", h, f)):
        a = torch.randn(PREFILL_TOKENS, k, device=dev, dtype=torch.bfloat16)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) for _ in range(4)]
        o = torch.empty(PREFILL_TOKENS, n, device=dev, dtype=torch.bfloat16)
        turn = [0]

        def one():
            torch.matmul(a, ws[turn[0] % 4].t(), out=o)
            turn[0] += 1
        for _ in range(5):
            one()
        us = timed(one, 30) * 1e3
        shapes[name] = {"us": round(us, 1), "tflops": round(2.0 * PREFILL_TOKENS * n * k / us / 1e6, 1)}
        del a, ws, o
    print(json.dumps({"only": "peaks", "copy_gbs": round(copy_gbs, 1), "bf16_tflops_burst": round(flop / burst_ms / 1e9, 1),
                      "bf16_tflops_loop": round(flop / loop_ms / 1e9, 1), "loop_reps": reps, "clocks": clk,
                      "library_on_prompt_shapes": shapes, "in_use": peaks()}))
    return 0


def prefill_slots(engine, slots, prompt_len, rng):
    """Run a prompt of ``prompt_len`` random token ids into every slot, one prompt a step (keeps the
    scratch memory of a step small)."""
    V = engine.spec.vocab_size
    for s in slots:
        engine.step([s], [rng.integers(0, V, size=prompt_len).tolist()], [[]])


def timed_decode(engine, sampler, slots, steps, warmup, rng, spread=None):
    """``steps`` decode steps of the sequences in ``slots`` (already holding their prompts), as
    generation runs them: the sampler draws from a step's logits (greedy, through ``Sampler``) and
    leaves the ids on the device, the next step takes them from there (``Engine.step_fed``), the ids
    also start on their way to the host.  Timed on the device between two events, no host wait
    inside.  Returns (ms, kernels launched, mean positions a sequence held during the timed steps)."""
    import torch
    from ultima_b200.sampling import SamplingParams
    from ultima_b200.sampling.sampler import stream_seed
    V = engine.spec.vocab_size
    B = len(slots)
    params = [SamplingParams()] * B
    streams = [stream_seed(0, i) for i in range(B)]
    state = {"n": 0, "pend": None, "logits": None}

    def one():
        if state["pend"] is None:
            logits = engine.step(slots, [[int(t)] for t in rng.integers(0, V, size=B)], None, borrow=True)
        else:
            logits = engine.step_fed(slots, state["pend"].ids_dev)
        state["pend"] = sampler.begin(logits, params, streams, [state["n"]] * B, None, continuing=state["n"] > 0)
        state["logits"] = logits
        state["n"] += 1
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    ctx0 = engine.length(slots[0])
    l0 = engine.rt.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = engine.rt.launches - l0 + steps            # the engine's kernels and one sampling kernel a step
    ids = state["pend"].wait()
    if not bool(torch.isfinite(state["logits"]).all()) or min(ids) < 0 or max(ids) >= V:
        raise RuntimeError("decode step gave logits that are not finite, or a token id outside the vocabulary")
    ctx = ctx0 + steps / 2
    if spread is not None:
        # how even the steps are: a few more of them, each between two events of its own
        n = min(32, steps)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        evs[0].record()
        for i in range(n):
            one()
            evs[i + 1].record()
        torch.cuda.synchronize()
        each = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(n))
        spread.update({"p10": round(each[n // 10], 4), "median": round(each[n // 2], 4),
                       "p90": round(each[(9 * n) // 10], 4), "steps": n})
    return ms, launches, ctx


def decode_timeline(engine, batch, prompt_len, rng):
    """Where the time of one decode step goes, kernel by kernel, as the step really runs (inside its
    captured graph, kernels overlapping through dependent launches): for each kernel of the step's
    last layers and the head, when it began and ended and how much later it ended than the kernel
    before it (the share of the step's time that is its own).  Timestamps come from CUPTI through
    torch.profiler; run few layers (--layers 6)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    V = engine.spec.vocab_size
    slots = engine.open(batch)
    fill_cache(engine, slots, prompt_len)

    def one():
        engine.step(slots, [[int(t)] for t in rng.integers(0, V, size=batch)], None, borrow=True)
    for _ in range(6):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    ev.sort(key=lambda e: e.time_range.start)
    last = ev[2 * (len(ev) // 3):]                       # the third step
    t0 = last[0].time_range.start
    rows, prev_end = [], None
    for e in last:
        s, en = e.time_range.start - t0, e.time_range.end - t0
        rows.append({"kernel": e.name.split("(")[0].replace("void ", "")[:48], "start_us": round(s, 2),
                     "end_us": round(en, 2), "own_us": None if prev_end is None else round(en - prev_end, 2)})
        prev_end = en if prev_end is None else max(prev_end, en)
    engine.close(slots)
    engine.check_errors()
    for r in rows[-24:]:
        print(json.dumps(r))
    print(json.dumps({"only": "timeline", "batch": batch, "layers": len(engine.spec.layers),
                      "kernels_a_step": len(last), "step_us": round(prev_end, 2)}))
    return 0


def prefill_timeline(engine, tokens, rng):
    """The same for one prompt of ``tokens`` tokens: the kernels of its last layers with begin, end and
    own share (run few layers: --layers 4)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    prompt = rng.integers(0, engine.spec.vocab_size, size=tokens).tolist()

    def one():
        s = engine.open(1)
        engine.step(s, [prompt], None)
        engine.close(s)
    for _ in range(3):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        one()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    ev.sort(key=lambda e: e.time_range.start)
    t0 = ev[0].time_range.start
    rows, prev_end = [], None
    for e in ev:
        s, en = e.time_range.start - t0, e.time_range.end - t0
        rows.append({"kernel": e.name.split("(")[0].replace("void ", "")[:48], "start_us": round(s, 2),
                     "end_us": round(en, 2), "own_us": None if prev_end is None else round(en - prev_end, 2)})
        prev_end = en if prev_end is None else max(prev_end, en)
    engine.check_errors()
    for r in rows[-20:]:
        print(json.dumps(r))
    print(json.dumps({"only": "timeline-prefill", "tokens": tokens, "layers": len(engine.spec.layers),
                      "kernels": len(ev), "prompt_us": round(prev_end, 2)}))
    return 0


def attention_times(lengths=(2048, 4096, 8192, 16384), nh=32, nkv=8, hd=128):
    """Device time of the prompt attention kernel alone (one sequence, causal, Qwen3-8B head counts), one
    JSON line a prompt length: microseconds a launch and TFLOP/s of the causal half."""
    import math
    import torch
    from ultima_b200.engine import Runtime
    from ultima_b200.kernels import attn_tc
    dev = torch.device("cuda:0")
    rt = Runtime(dev, torch.bfloat16)

    class Box:
        pass
    for T in lengths:
        pages = (T + 63) // 64
        kv = Box()
        kv.k = torch.randn(pages, nkv, 64, hd, device=dev).to(torch.bfloat16)
        kv.v = torch.randn(pages, nkv, 64, hd, device=dev).to(torch.bfloat16)
        kv.table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1)
        kv.ring, kv.page, kv.window = pages * 64, 64, None
        q = torch.randn(T, nh * hd, device=dev).to(torch.bfloat16)
        out = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=dev)
        b = Box()
        b.seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
        b.seq_before = torch.tensor([0], dtype=torch.int32, device=dev)
        b.n_seqs, b.max_new, b.max_after = 1, T, T
        def run():
            attn_tc.attention(q, kv, out, b, nh, nkv, hd, 1 / math.sqrt(hd), rt)
        for _ in range(3):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            run()
        e1.record()
        torch.cuda.synchronize()
        rt.check_status()
        us = e0.elapsed_time(e1) / 20 * 1e3
        print(json.dumps({"only": "attention", "tokens": T, "heads": nh, "kv_heads": nkv, "head_dim": hd,
                          "us": round(us, 1), "tflops_causal": round(4 * nh * hd * (T * (T + 1) / 2) / us / 1e6, 1)}))
    return 0


def sampling_times(batches=(1, 8, 64), vocab=151936, history=256):
    """Device time of the sampling kernel alone at the 8B vocabulary, for the reference's ladder
    of options (src/sampler/sampler.cpp:230-277): one JSON line a batch size, microseconds a call.
    Rows use rings of recent tokens on the device as the generation loop does."""
    import dataclasses
    import numpy as np
    import torch
    from ultima_b200.engine import Runtime
    from ultima_b200.kernels import ops
    from ultima_b200.sampling import Sampler, SamplingParams
    dev = torch.device("cuda:0")
    rt = Runtime(dev, torch.bfloat16)
    server = SamplingParams.server_defaults()
    modes = [("greedy", SamplingParams()), ("temperature", SamplingParams(temperature=0.8)),
             ("top_k 40", SamplingParams(temperature=0.8, top_k=40)),
             ("top_p 0.9", SamplingParams(temperature=0.8, top_p=0.9)),
             ("min_p 0.05", SamplingParams(temperature=0.8, min_p=0.05)),
             ("greedy + repetition penalty", SamplingParams(rep_penalty=1.1, repeat_last_n=64)),
             ("server defaults without penalties", dataclasses.replace(server, rep_penalty=1.0, dry_multiplier=0.0)),
             ("server defaults", server)]
    rng = np.random.default_rng(0)
    for B in batches:
        logits = torch.randn(B, vocab, device=dev) * 3
        row = {"only": "sample", "batch": B, "vocab": vocab, "unit": "us a call, kernel only"}
        for name, sp in modes:
            smp = Sampler(dev, vocab, rt)
            hs = [rng.integers(0, vocab, size=history).tolist() for _ in range(B)]
            for step in range(3):                    # as the loop does: the drawn token joins the history
                ids = smp.sample(logits, [sp] * B, list(range(B)), [step] * B, hs)
                for h, t in zip(hs, ids):
                    h.append(t)
            _, _, _, rec_dev, bid, bval, _ = smp._cache
            out = torch.empty(B, dtype=torch.int32, device=dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for i in range(20):
                ops.sample(logits, smp._work, rec_dev, smp._dummy_i, bid if bid is not None else smp._dummy_i,
                           bval if bval is not None else smp._dummy_f, out, 3 + i, smp._hist, smp._hist_len)
            e1.record()
            torch.cuda.synchronize()
            row[name] = round(e0.elapsed_time(e1) / 20 * 1e3, 1)
        print(json.dumps(row))
    return 0


def run_ours(args):
    import numpy as np
    import torch
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.engine.generate import LoopStats, generate
    from ultima_b200.sampling import Sampler, SamplingParams
    from ultima_b200.weights import random_tensors_on_device

    pk = peaks()
    d = dict(QWEN3_8B)
    layers_full = d["num_hidden_layers"]
    if args.layers:
        d["num_hidden_layers"] = args.layers
    cfg = u.config_from_dict(d)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    spec = u.model_spec_for(cfg)
    t0 = time.time()
    tensors = random_tensors_on_device(spec.weight_specs(), 0, torch.bfloat16, dev)
    run = args.warmup + args.steps
    whole = args.only == "all"
    # the far end of the metric: prompts long enough that three timed runs (batch 64, 8, 1, one after
    # another on the same sequences) end just below the context of 8,192 positions
    far_prompt = (CONTEXT - 3 * run - 40) // 64 * 64
    if whole and far_prompt < PROMPT:
        raise SystemExit(f"bench.py: --steps {args.steps} leaves no room for the points near {CONTEXT} positions")
    if whole:
        n_seq, per_seq = 64, CONTEXT
    else:
        n_seq = args.batch
        per_seq = -(-(max(args.prompt, PROMPT) + run + 64) // 64) * 64
    engine = Engine(spec, tensors, dtype="bfloat16", max_tokens=max(n_seq * per_seq, args.prefill_tokens + 64),
                    max_seqs=n_seq, max_step_tokens=max(PREFILL_TOKENS, min(args.prefill_tokens, 8192)),
                    max_context=max(CONTEXT, args.prompt + run + 64, args.prefill_tokens))
    del tensors
    sampler = Sampler(dev, cfg.vocab_size, engine.rt)
    rng = np.random.default_rng(0)
    engine.warm_up()
    print(f"[bench] model ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)

    if args.only == "timeline":
        return decode_timeline(engine, args.batch, args.prompt, rng)
    if args.only == "timeline-prefill":
        return prefill_timeline(engine, args.prefill_tokens, rng)

    wbytes = weight_bytes(cfg)
    kvb = kv_bytes_per_token(cfg, 2)

    def frac_of(batch, ctx, ms_step):
        return (wbytes + batch * ctx * kvb) / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"]

    if args.only == "decode":
        slots = engine.open(args.batch)
        if args.fast_fill:
            fill_cache(engine, slots, args.prompt)
        else:
            prefill_slots(engine, slots, args.prompt, rng)
        ms, launches, ctx = timed_decode(engine, sampler, slots, args.steps, args.warmup, rng)
        engine.close(slots)
        engine.check_errors()
        print(json.dumps({"only": "decode", "batch": args.batch, "layers": cfg.num_hidden_layers,
                          "ms_per_step": round(ms / args.steps, 4), "context": int(ctx),
                          "hbm_frac": round(frac_of(args.batch, ctx, ms / args.steps), 4),
                          "value": round(args.batch * args.steps / ms * 1e3, 1), "gpu_launches": int(launches)}))
        return 0

    # prefill of one 2,048-token prompt
    PT = args.prefill_tokens
    prompt = rng.integers(0, cfg.vocab_size, size=PT).tolist()
    pre_ms = []
    for i in range(2 + 3):
        s = engine.open(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step(s, [prompt], None)
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i >= 2:
            pre_ms.append(e0.elapsed_time(e1))
    pms = statistics.median(pre_ms)
    pf = prefill_flops(cfg, PT)
    prefill = {"value": round(PT / pms * 1e3, 1), "tokens": PT, "ms": round(pms, 3),
               "frac": round(pf / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               # the same against what a long run of products holds under the power cap
               "frac_sustained": round(pf / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
    print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)
    if args.only == "prefill":
        engine.check_errors()
        print(json.dumps({"only": "prefill", "layers": cfg.num_hidden_layers, **prefill}))
        return 0

    # the headline: batch 8 from 2,048-token prompts
    slots = engine.open(BATCH)
    prefill_slots(engine, slots, PROMPT, rng)
    clocks = ClockSampler()
    clocks.start()
    spread = {}
    ms, launches, ctx = timed_decode(engine, sampler, slots, args.steps, args.warmup, rng, spread=spread)
    clk = clocks.stop()
    engine.close(slots)
    value = BATCH * args.steps / ms * 1e3
    achieved = (wbytes + BATCH * ctx * kvb) / (ms / args.steps * 1e-3) / 1e9
    print(f"[bench] decode b{BATCH}: {value:.1f} tok/s", file=sys.stderr, flush=True)

    # the other points: 64 sequences that have really run their prompts, then 8 and 1 of the same
    # sequences; first from 2,048-token prompts, then near the end of the context
    points, point_frac, point_ctx = {}, {}, {}
    for tag, plen, batches in (("", PROMPT, (64, 1)), ("_ctx8k", far_prompt, (64, 8, 1))):
        slots = engine.open(64)
        tp = time.time()
        prefill_slots(engine, slots, plen, rng)
        torch.cuda.synchronize()
        print(f"[bench] 64 prompts of {plen} tokens in {time.time() - tp:.1f} s", file=sys.stderr, flush=True)
        for b in batches:
            engine.close(slots[b:])
            slots = slots[:b]
            pm, _, pctx = timed_decode(engine, sampler, slots, args.steps, args.warmup, rng)
            key = f"decode_b{b}{tag}"
            points[key] = round(b * args.steps / pm * 1e3, 1)
            point_frac[key] = round(frac_of(b, pctx, pm / args.steps), 4)
            point_ctx[key] = int(pctx)
            print(f"[bench] {key}: {points[key]} tok/s at {int(pctx)} positions, {point_frac[key]} of the copy bandwidth",
                  file=sys.stderr, flush=True)
        engine.close(slots)

    # end to end through the generation loop: host token ids in, sampled ids out, every step
    prompts = [rng.integers(0, cfg.vocab_size, size=PROMPT).tolist() for _ in range(BATCH)]
    stats = LoopStats()
    n_new = args.warmup + args.steps + 1         # the prompts' own token, then warm-up steps, then the timed steps
    generate(engine, sampler.sample, prompts, SamplingParams(), n_new, (), max_batch=BATCH, stats=stats)
    stats = LoopStats()
    generate(engine, sampler.sample, prompts, SamplingParams(), n_new, (), max_batch=BATCH, stats=stats)
    # the same rule as for ``value``: the first ``warmup`` steps after the prompts are not timed, then exactly
    # ``steps`` steps are, on the host's clock from the arrival of one step's ids to the arrival of the last's
    done = stats.step_done_s
    assert len(done) == n_new and args.steps < len(done)
    e2e_val = BATCH * args.steps / (done[-1] - done[-1 - args.steps])
    h2d = engine.last_h2d_bytes                   # the step's record (ids, positions, page tables); the
    # sampler's records stay on the device while a batch samples with the same parameters
    dev_ms = sorted(stats.device_step_ms)
    e2e = {"value": round(e2e_val, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
           "d2h_bytes_per_step": 4 * (BATCH + 4),          # the sampled ids and the kernels' status flags
           "device_ms_per_step": round(dev_ms[len(dev_ms) // 2], 4) if dev_ms else None}

    engine.check_errors()
    out = {
        "metric": "decode tokens/s, Qwen3-8B sizes, bf16, batch 8, 2048-token prompts",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights from a seed, random token ids",
        "config": {"model": "Qwen3-8B sizes", "layers": cfg.num_hidden_layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT, "decode_context": int(ctx),
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (15 GB of weights a step)",
                   "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clk, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_hbm_frac": point_frac, "points_context": point_ctx, "step_ms": spread, "impl": "ours",
    }
    print(json.dumps(out), flush=True)
    return 0


def run_other(args):
    """Qwen3-14B / Qwen3-32B layer sizes: a batch of prompts (run one after another), then decode steps."""
    import numpy as np
    import torch
    import ultima_b200 as u
    from ultima_b200.engine import Engine
    from ultima_b200.sampling import Sampler
    from ultima_b200.weights import random_tensors_on_device
    w = OTHER[args.config]
    pk = peaks()
    d = dict(QWEN3_8B)
    d.update(w["sizes"])
    if args.layers:
        d["num_hidden_layers"] = args.layers
    cfg = u.config_from_dict(d)
    dev = torch.device("cuda:0")
    spec = u.model_spec_for(cfg)
    rng = np.random.default_rng(0)
    kind, lo, hi = w["prompt"]
    B, steps = w["batch"], (args.steps if args.steps_given else w["decode"])
    lens = [int(x) for x in (rng.integers(lo, hi + 1, size=B) if kind == "uniform" else [hi] * B)]
    per_seq = [-(-(n + steps + 8) // 64) * 64 for n in lens]
    engine = Engine(spec, random_tensors_on_device(spec.weight_specs(), 0, torch.bfloat16, dev), dtype="bfloat16",
                    max_tokens=sum(per_seq), max_seqs=B, max_step_tokens=4096, max_context=CONTEXT)
    sampler = Sampler(dev, cfg.vocab_size, engine.rt)
    engine.warm_up()
    print(f"[bench] {args.config}: model ready", file=sys.stderr, flush=True)
    slots = engine.open(B)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in lens]
    engine.step([slots[0]], [prompts[0][:64]], [[]])            # warm the prompt kernels
    engine.close([slots[0]])
    slots[0] = engine.open(1)[0]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(B):
        engine.step([slots[i]], [prompts[i]], [[]])
    e1.record()
    torch.cuda.synchronize()
    pre_ms = e0.elapsed_time(e1)
    print(f"[bench] {args.config}: {sum(lens)} prompt tokens in {pre_ms:.1f} ms", file=sys.stderr, flush=True)
    clocks = ClockSampler()
    clocks.start()
    ms, _, _ = timed_decode(engine, sampler, slots, steps, args.warmup, rng)
    clk = clocks.stop()
    print(f"[bench] {args.config}: {steps} decode steps in {ms:.1f} ms", file=sys.stderr, flush=True)
    engine.check_errors()
    mean_ctx = sum(lens) / B + args.warmup + steps / 2
    step_bytes = weight_bytes(cfg) + B * mean_ctx * kv_bytes_per_token(cfg, 2)
    achieved = step_bytes / (ms / steps * 1e-3) / 1e9
    pf = sum(prefill_flops(cfg, n) for n in lens)
    print(json.dumps({
        "metric": f"decode tokens/s, Qwen3-{args.config.upper()} sizes, bf16, batch {B}", "value": round(B * steps / ms * 1e3, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": round(ms / steps, 4),
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic: random weights from a seed, random token ids",
        "config": {"model": f"Qwen3-{args.config.upper()} sizes", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": B,
                   "prompt_tokens": sum(lens), "prompt_min": min(lens), "prompt_max": max(lens), "peaks": pk["source"]},
        "prefill": {"value": round(sum(lens) / pre_ms * 1e3, 1), "tokens": sum(lens), "ms": round(pre_ms, 2),
                    "frac": round(pf / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clk, "impl": "ours"}), flush=True)
    return 0


REF_MODEL_SRCS = ["dtype", "tensor_info", "metadata_store", "loaded_model", "arch_registry", "qwen_config",
                  "qwen_tensor_slots", "weight_dispatch", "qwen_block", "qwen_model", "hadamard"]
REF_LAYERS = 2            # of the 36: what the reference's CPU code gets through in about a minute
REF_PROMPT, REF_PREFILL_TOKENS = 64, 256


def build_reference(say) -> str:
    """The reference's own sources, copied unchanged into baseline/_ref/src and compiled there with g++
    for the CPU (its CMake build fetches packages from the network and its file loader is for Windows
    only, so the translation units of the model path are compiled directly), linked with
    baseline/ref_bench.cpp.  Returns the program's path, or raises with the reason."""
    import glob
    import shutil
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    exe = os.path.join(ref_root, "ref_bench")
    harness = os.path.join(ROOT, "baseline", "ref_bench.cpp")
    if os.path.isfile(exe) and os.path.getmtime(exe) >= os.path.getmtime(harness):
        return exe
    src = os.environ.get("ULTIMA_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isfile(os.path.join(src, "src", "model", "qwen_model.cpp")):
        raise RuntimeError("the reference's sources are not on this machine and no program was built before "
                           "(set ULTIMA_REFERENCE_DIR to a checkout of tattooinmtl/Ultima.cpp)")
    if not shutil.which("g++"):
        raise RuntimeError("no g++ to compile the reference's sources with")
    tree = os.path.join(ref_root, "src_tree")
    for sub in ("include", "src"):
        dst = os.path.join(tree, sub)
        if not os.path.isdir(dst):
            shutil.copytree(os.path.join(src, sub), dst)
    inc = os.path.join(ref_root, "inc")
    os.makedirs(os.path.join(inc, "nonstd"), exist_ok=True)
    os.makedirs(os.path.join(ref_root, "obj"), exist_ok=True)
    import torch
    if not os.path.exists(os.path.join(inc, "fmt")):        # the header-only fmt inside the torch wheel, as a formatting library
        shutil.copytree(os.path.join(os.path.dirname(torch.__file__), "include", "fmt"), os.path.join(inc, "fmt"))
    with open(os.path.join(inc, "nonstd", "expected.hpp"), "w") as f:
        f.write("#pragma once\n#include <expected>\nnamespace nonstd { using std::expected; using std::unexpected; }\n")
    srcs = ["src/core/error.cpp", "src/runtime/thread_pool.cpp", "src/kv_cache/kv_cache.cpp",
            "src/kv_cache/recurrent_state.cpp", "src/sampler/sampler.cpp"]
    srcs += sorted(os.path.relpath(q, tree) for q in glob.glob(os.path.join(tree, "src/kernels/*.cpp")))
    srcs += [f"src/model/{m}.cpp" for m in REF_MODEL_SRCS]
    flags = ["-std=c++23", "-O2", "-mavx2", "-mfma", "-DFMT_HEADER_ONLY", "-include", "immintrin.h",
             "-I", os.path.join(tree, "include"), "-I", os.path.join(tree, "src/model"), "-isystem", inc]
    say(f"compiling {len(srcs)} files of the reference with g++ ...")
    procs = []
    for q in srcs:
        obj = os.path.join(ref_root, "obj", q.replace("/", "_") + ".o")
        if not os.path.exists(obj):
            procs.append(subprocess.Popen(["g++"] + flags + ["-c", os.path.join(tree, q), "-o", obj]))
        if len(procs) >= 8:
            if any(pr.wait() != 0 for pr in procs):
                raise RuntimeError("g++ failed on the reference's sources")
            procs = []
    if any(pr.wait() != 0 for pr in procs):
        raise RuntimeError("g++ failed on the reference's sources")
    objs = sorted(glob.glob(os.path.join(ref_root, "obj", "*.o")))
    if subprocess.call(["g++"] + flags + [harness] + objs + ["-lpthread", "-o", exe]) != 0:
        raise RuntimeError("g++ failed on baseline/ref_bench.cpp")
    return exe


def run_reference(args):
    """The reference arm: the reference's unmodified model code through its own public interface, on the
    CPU it is written for (it has no GPU code), same metric and unit.  It has no batch, so the eight
    sequences of a step run one after another; it runs REF_LAYERS of the 36 layers, from prompts of
    REF_PROMPT tokens, and both are named in ``config``.  When neither a program built before nor the
    sources and a compiler are there, the line says ``unavailable`` with the reason."""
    def say(msg):
        print(f"[bench] {msg}", file=sys.stderr, flush=True)
    try:
        exe = build_reference(say)
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}), flush=True)
        return 0
    c = QWEN3_8B
    steps = args.steps if args.steps is not None else 16
    warmup = max(1, min(args.warmup, 3))
    threads = os.cpu_count() or 1
    cmd = [exe] + [str(x) for x in (REF_LAYERS, c["hidden_size"], c["intermediate_size"], c["num_attention_heads"],
                                    c["num_key_value_heads"], c["head_dim"], c["vocab_size"], BATCH, REF_PROMPT, steps,
                                    warmup, REF_PREFILL_TOKENS, threads)]
    say("running " + " ".join(cmd[1:]))
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=1400)
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's program did not end within its time limit"}), flush=True)
        return 0
    if res.returncode != 0 or not res.stdout.strip():
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's program ended with code {res.returncode}: "
                          + res.stderr.strip()[-200:]}), flush=True)
        return 0
    dec, pre, ms_step, pre_ms = (float(x) for x in res.stdout.split())
    out = {
        "metric": "decode tokens/s, Qwen3-8B sizes, bf16, batch 8, 2048-token prompts",
        "value": round(dec, 3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights, fp32 arithmetic (the reference's only arithmetic)",
        "data": "synthetic: random weights from a hash, token ids from a hash",
        "config": {"model": "Qwen3-8B sizes", "layers": REF_LAYERS, "layers_full": c["num_hidden_layers"],
                   "hidden": c["hidden_size"], "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
                   "head_dim": c["head_dim"], "intermediate": c["intermediate_size"], "vocab": c["vocab_size"],
                   "global_batch": BATCH, "batching": "none: the sequences of a step one after another",
                   "prompt_len": REF_PROMPT, "device": "cpu", "threads": threads, "parallelism": "the host's cores"},
        # the reference's interface is the host's: token ids in, logits out, its own argmax; nothing is copied
        "e2e": {"value": round(dec, 3), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "prefill": {"value": round(pre, 2), "tokens": REF_PREFILL_TOKENS, "ms": round(pre_ms, 2)},
        "impl": "reference",
    }
    print(json.dumps(out), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--config", default="8b", choices=["8b", "14b", "32b"],
                    help="8b: the default run; 14b, 32b: the baseline's other two workloads")
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "timeline", "timeline-prefill", "sample", "attention", "peaks"],
                    help="a part of the run only (for profiling); the JSON line then holds that part. "
                         "timeline: every kernel of a decode step with its begin and end inside the graph "
                         "(timeline-prefill: of a prompt); "
                         "sample: the sampling kernel alone, option by option; attention: the prompt attention alone; "
                         "peaks: this GPU's copy bandwidth and library bfloat16 product, the denominators' kind")
    ap.add_argument("--batch", type=int, default=BATCH, help="sequences of the decode step")
    ap.add_argument("--fast-fill", action="store_true", help="do not run the prompts; mark the cache as filled")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="positions each sequence holds before the timed steps")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="tokens of the timed prompt")
    ap.add_argument("--watchdog", type=int, default=1500,
                    help="seconds after which a run that has not ended dumps its stack and exits (0: never)")
    args = ap.parse_args()
    if args.watchdog > 0:
        # a run that stops making progress ends with a message instead of holding its GPU
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 64
    if args.only == "sample":
        return sampling_times()
    if args.only == "attention":
        return attention_times()
    if args.only == "peaks":
        return measured_peaks()
    if args.config != "8b":
        return run_other(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
