"""The generation loop above the step function, and the Python entry point.

The loop is the reference's (apps/ultima-cli/main.cpp:652-686; server flavour
src/server/http_server.cpp:158-202) for a batch: prefill, then repeat {sample from the
current logits; stop check; emit; decode}.  A stop token is neither emitted nor fed back
(main.cpp:675); nothing is decoded after the last sampled token (http_server.cpp:196); a
request whose prompt and new tokens would not fit the context is refused before anything
runs (main.cpp:637-641).  Requests are run in batches of sequences that start together;
a sequence that ends leaves the batch and gives its slot back at once, and batches follow
one another until every request is done.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..cache.book import PAGE
from ..sampling.params import SamplingParams
from ..sampling.sampler import stream_seed


@dataclass
class Generation:
    tokens: list
    finish_reason: str          # "stop" (a stop token was sampled), "length", "context"
    prompt_len: int = 0


@dataclass
class LoopStats:
    """What a run of the loop cost.  ``prefill_s`` and ``decode_s`` are the host's clock, as the
    reference reports them (apps/ultima-cli/main.cpp:689-698); ``device_prefill_ms`` and
    ``device_step_ms`` are the device's own time of the prompt step and of every decode step
    (between marks the engine leaves on the stream), where the engine can give marks."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_s: float = 0.0
    decode_s: float = 0.0
    steps: int = 0
    device_prefill_ms: float = 0.0
    device_step_ms: list = field(default_factory=list)
    step_done_s: list = field(default_factory=list)       # the host's clock when each step's ids had arrived


def plan_batches(prompt_lens: list, max_batch: int, max_tokens: int, n_predict: list, page: int = PAGE):
    """Requests in order, cut into batches of at most ``max_batch`` whose tokens (prompt plus
    what may be generated, each rounded up to a page) fit ``max_tokens``."""
    def cost(i):
        return -(-(prompt_lens[i] + n_predict[i]) // page) * page
    batches, cur, used = [], [], 0
    for i in range(len(prompt_lens)):
        c = cost(i)
        if c > max_tokens:
            raise ValueError(f"request {i} needs {c} cache positions; the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or used + c > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += c
    if cur:
        batches.append(cur)
    return batches


def run_batch(engine, sample, prompts: list, params: list, n_predict: list, stop_ids, streams: list,
              max_context: int, stats: LoopStats | None = None) -> list:
    """One batch from its prompts to its last token.

    engine: has open(n), close(slots), step(slots, tokens, want) -> logits rows
    sample(logits, params, streams, counters, recents) -> list of token ids
    """
    n = len(prompts)
    stop = set(int(s) for s in stop_ids)
    out = [Generation([], "length", len(p)) for p in prompts]
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i} has an empty prompt")
        if len(p) + n_predict[i] > max_context:
            raise ValueError(f"request {i}: prompt of {len(p)} plus {n_predict[i]} new tokens "
                             f"does not fit the context of {max_context}")
    # what the penalties look back on: the prompt, then what was generated (the reference pushes the
    # prompt's tokens into its sampler's window before the first draw, apps/ultima-cli/main.cpp:664,
    # src/server/http_server.cpp:163); built only for requests whose parameters read it
    seen = [list(p) if params[i].uses_history else [] for i, p in enumerate(prompts)]
    slots = engine.open(n)
    held = set(range(n))
    try:
        live = [i for i in range(n) if n_predict[i] > 0]
        for i in range(n):
            if n_predict[i] <= 0:
                engine.close([slots[i]])
                held.discard(i)
        if not live:
            return out
        t0 = time.perf_counter()
        borrow = {"borrow": True} if getattr(engine, "use_graphs", False) else {}
        # A sampler that can hand its token ids on without the host (begin / wait) and an engine that
        # can take them from the device (step_fed) let the next step be queued before this step's ids
        # have reached the host: the device then never waits for the host between two steps.
        owner = getattr(sample, "__self__", None)
        begin = getattr(sample, "begin", None) or getattr(owner, "begin", None)
        ahead = begin is not None and getattr(engine, "feeds_from_device", False)
        mark = getattr(engine, "mark", None) if stats is not None else None
        marks = [mark()] if mark else []
        logits = engine.step([slots[i] for i in live], [prompts[i] for i in live], None)
        if mark:
            marks.append(mark())
        if stats:
            stats.prompt_tokens += sum(len(prompts[i]) for i in live)

        def draw(rows_logits, rows, continuing=False):
            args = (rows_logits, [params[i] for i in rows], [streams[i] for i in rows],
                    [len(out[i].tokens) for i in rows], [seen[i] for i in rows])
            if begin is None:
                ids = sample(*args)
                return lambda: ids
            return begin(*args, continuing=continuing).wait

        first = True
        pending = draw(logits, live)
        while live:
            # queue the next step now if every sequence goes on unless it draws a stop token
            next_logits = None
            if ahead and all(len(out[i].tokens) + 1 < n_predict[i] for i in live):
                ids_dev = getattr(getattr(pending, "__self__", None), "ids_dev", None)
                if ids_dev is not None:
                    next_logits = engine.step_fed([slots[i] for i in live], ids_dev)
                    if mark:
                        marks.append(mark())
            ids = pending()
            now = time.perf_counter()
            if stats:
                if first:
                    stats.prefill_s += now - t0
                else:
                    stats.decode_s += now - t0
                stats.steps += 1
                stats.step_done_s.append(now)
            first = False
            t0 = now
            going, feed, rows = [], [], []
            for r, (i, tok) in enumerate(zip(live, ids)):
                tok = int(tok)
                if params[i].uses_history:
                    seen[i].append(tok)
                if tok in stop:
                    out[i].finish_reason = "stop"
                elif len(out[i].tokens) + 1 >= n_predict[i]:
                    out[i].tokens.append(tok)
                    out[i].finish_reason = "length"
                else:
                    out[i].tokens.append(tok)
                    going.append(i)
                    feed.append([tok])
                    rows.append(r)
                    continue
                engine.close([slots[i]])            # a sequence that ends gives its slot back
                held.discard(i)
            same = going == live
            live = going
            if not live:
                break
            if next_logits is not None:
                # the step has run for all that were alive; those that stopped are dropped from its rows
                pending = draw(next_logits if same else next_logits[rows], live, continuing=same)
            else:
                logits = engine.step([slots[i] for i in live], feed, None, **borrow)
                if mark:
                    marks.append(mark())
                pending = draw(logits, live)
        return out
    finally:
        if stats:
            stats.generated_tokens += sum(len(g.tokens) for g in out)
            if len(marks) >= 2:
                # a mark after every step: the prompt step, then one decode step (and the sampling
                # of the step before it) between each two
                ms = [engine.elapsed_ms(a, b) for a, b in zip(marks[:-1], marks[1:])]
                stats.device_prefill_ms += ms[0]
                stats.device_step_ms.extend(ms[1:])
        if held:
            engine.close([slots[i] for i in sorted(held)])


def generate(engine, sample, prompts: list, params, n_predict, stop_ids=(), seed: int = 0,
             max_batch: int = 64, max_tokens: int | None = None, max_context: int | None = None,
             stats: LoopStats | None = None) -> list:
    """All requests, batch after batch.  ``params`` and ``n_predict`` may be one value for all
    requests or a list.  A sequence's random stream is keyed by ``seed`` and its index among
    the requests, so its tokens do not depend on how the requests were batched."""
    n = len(prompts)
    plist = list(params) if isinstance(params, (list, tuple)) else [params] * n
    nlist = list(n_predict) if isinstance(n_predict, (list, tuple)) else [int(n_predict)] * n
    if len(plist) != n or len(nlist) != n:
        raise ValueError("one SamplingParams and one n_predict for each prompt (or one for all)")
    for p in plist:
        p.validate()
    max_tokens = max_tokens if max_tokens is not None else engine.max_tokens
    max_context = max_context if max_context is not None else engine.max_context
    streams = [stream_seed(plist[i].seed if plist[i].seed else seed, i) for i in range(n)]
    results = [None] * n
    for batch in plan_batches([len(p) for p in prompts], max_batch, max_tokens, nlist):
        got = run_batch(engine, sample, [prompts[i] for i in batch], [plist[i] for i in batch],
                        [nlist[i] for i in batch], stop_ids, [streams[i] for i in batch],
                        max_context, stats)
        for i, g in zip(batch, got):
            results[i] = g
    return results


class LLM:
    """The Python entry point: a model folder in, token ids in and out.

        llm = LLM("model_dir", dtype="bfloat16", n_ctx=512)
        outs = llm.generate([[1, 2, 3], [4, 5]], n_predict=48, temp=0.0, seed=0)

    Option names follow the reference's ``run`` command where it has them (n_predict, n_ctx,
    temp, seed; apps/ultima-cli/main.cpp:561-584) and its sampler's fields for the rest.
    """

    def __init__(self, model_dir: str, dtype: str = "bfloat16", n_ctx: int = 512, max_batch: int = 64,
                 max_tokens: int | None = None, device: str = "cuda:0", **engine_kw):
        from .engine import Engine
        from ..sampling.sampler import Sampler
        self.max_batch = int(max_batch)
        if max_tokens is None:
            max_tokens = self.max_batch * (-(-int(n_ctx) // PAGE) * PAGE)
        self.engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=max_tokens, max_context=n_ctx,
                                      max_seqs=self.max_batch, device=device, **engine_kw)
        self.sampler = Sampler(self.engine.device, self.engine.spec.vocab_size, self.engine.rt)
        self.stop_token_ids = tuple(self.engine.spec.stop_token_ids)
        self.last_stats = None

    def generate(self, prompts, n_predict: int = 48, temp: float = 0.0, seed: int = 0,
                 stop_token_ids=None, sampling: SamplingParams | list | None = None) -> list:
        """prompts: a list of token-id lists (or one list).  Returns a Generation for each."""
        single = bool(prompts) and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        if sampling is None:
            sampling = SamplingParams(temperature=float(temp))
        stop = self.stop_token_ids if stop_token_ids is None else tuple(stop_token_ids)
        self.last_stats = LoopStats()
        res = generate(self.engine, self.sampler.sample, [list(map(int, p)) for p in prompts], sampling,
                       n_predict, stop, seed=seed, max_batch=self.max_batch, stats=self.last_stats)
        return res[0] if single else res

    # the step function and the slots of the engine underneath, for callers that drive it themselves
    def step(self, slots, tokens, want=None):
        return self.engine.step(slots, tokens, want)

    def acquire(self, n: int = 1) -> list:
        return self.engine.open(n)

    def release(self, slots) -> None:
        self.engine.close(slots)


def load(model_dir: str, dtype: str = "bfloat16", max_ctx: int = 512, max_batch: int = 64, **kw) -> LLM:
    """Load a model folder; the same as ``LLM(model_dir, dtype=dtype, n_ctx=max_ctx, max_batch=max_batch)``."""
    return LLM(model_dir, dtype=dtype, n_ctx=max_ctx, max_batch=max_batch, **kw)
