"""The step function: a batch of sequences that started together, with unequal lengths;
their prompts in one step, then one token each.

``Engine.step`` runs only the tokens it is given, as one batch, from what earlier steps left
in the cache, and returns float32 logits at the wanted places.  The reference has two calls
on one sequence, prefill and decode, both one function underneath "because two code paths
would be two chances for them to disagree" (include/ultima/model/qwen_block.hpp:104-107,
src/model/qwen_model.cpp:80-141); here the same holds for a whole ragged batch: prompts and
single tokens go through the same kernels.  Long prompts are cut into several passes inside
a step (the reference cuts them into chunks of 32, src/model/qwen_model.cpp:104-117); the
cut changes no result beyond rounding.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import arch as _arch  # noqa: F401  (the architectures enter the registry when this is imported)
from ..cache import Cache, CacheError, PAGE
from ..config.base import config_from_dir, find_architecture
from ..parts.base import KVNeed, ModelSpec
from ..weights import load_weights
from .batch import DecodeRecord, PinnedRing, build_step_batch
from .model import Model
from .runtime import Runtime


class StepError(ValueError):
    """A step that cannot run: bad token ids, slots, positions; nothing was launched."""


def _dtype_of(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}[str(name)]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


class Engine:
    """A model on one GPU with its cache.

    max_tokens       positions that live sequences may hold together, each sequence rounded up
                     to a page of 64; sizes the cache
    max_seqs         slots (sequences alive at once)
    max_step_tokens  tokens of one pass through the layers; longer steps are cut into passes
    """

    def __init__(self, spec: ModelSpec, tensors: dict, dtype="bfloat16", max_tokens: int = 4096,
                 max_seqs: int | None = None, max_step_tokens: int = 4096, device="cuda:0",
                 max_context: int | None = None, poison_cache: bool = False, runtime=None,
                 use_graphs: bool = True, with_sampler: bool = True):
        self.spec = spec
        self.dtype = _dtype_of(dtype)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; the engine has no CPU path")
        torch.cuda.set_device(self.device)
        self.rt = runtime or Runtime(self.device, self.dtype)
        from ..kernels import build as _build, catalog as _catalog
        self.model = Model(spec, tensors, self.rt)        # parts refuse sizes no kernel takes here, before anything is compiled
        _build.prebuild(_catalog.targets_for_model(spec, self.dtype, sampler=with_sampler))     # nvcc runs side by side
        self.max_tokens = int(max_tokens)
        self.max_context = int(min(max_context or spec.max_positions, spec.max_positions))
        self.max_step_tokens = int(max_step_tokens)
        n_slots = int(max_seqs) if max_seqs else max(1, min(1024, -(-self.max_tokens // PAGE)))
        needs = self.model.cache_needs()
        windows = [n.window for need in needs for n in (need if isinstance(need, tuple) else (need,))
                   if isinstance(n, KVNeed) and n.window is not None]
        # a sequence brings at most this many tokens in one pass; with windows it also
        # bounds the span a windowed group must hold
        self.seq_chunk = self.max_step_tokens if not windows else min(self.max_step_tokens, 1024)
        self.cache = Cache(needs, self.model.cache_sources(), self.max_tokens, self.max_context,
                           n_slots, self.seq_chunk, dtype=self.rt.cache_dtype, device=self.device,
                           poison=poison_cache)
        self._ring = PinnedRing(self.device)
        self.last_h2d_bytes = 0
        # decode steps (one token a sequence, every logit wanted) are captured as CUDA graphs,
        # one for each (number of sequences, slices of the key range); parts must allow it
        from .model import TRACE as _tracing
        self.use_graphs = bool(use_graphs) and not _tracing and all(L.graph_safe for L in self.model.layers)
        self._graphs: dict = {}

    # ---- construction ------------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", **kw) -> "Engine":
        """Model class by config.json, weights by name from model.safetensors."""
        cfg = config_from_dir(model_dir)              # an ArchitectureConfig (config/base.py)
        entry = find_architecture(cfg.architecture)
        max_ctx = kw.get("max_context")
        # positions beyond what the cache can hold are never reached: size tables to that
        reach = min(cfg.max_position_embeddings, max_ctx or cfg.max_position_embeddings,
                    -(-int(kw.get("max_tokens", 4096)) // PAGE) * PAGE)
        spec = entry.build_spec(cfg, max_positions=reach)
        device = kw.get("device", "cuda:0")
        optional = ("lm_head.weight",) if spec.head.get("tied") else ()
        tensors = load_weights(model_dir, spec.weight_specs(), _dtype_of(dtype), device, optional)
        eng = cls(spec, tensors, dtype=dtype, **kw)
        eng.config = cfg
        return eng

    def warm_up(self) -> None:
        """Compile and load every kernel this model uses by running one short sequence."""
        s = self.open(1)
        try:
            self.step(s, [[0, 0, 0]], [[2]])
            self.step(s, [[0]], [[0]])
            torch.cuda.synchronize(self.device)
        finally:
            self.close(s)

    def check_errors(self) -> None:
        """Raise if a kernel flagged a fault since the last check (waits for the stream)."""
        self.rt.check_status()

    # ---- slots -------------------------------------------------------------------------
    def open(self, n: int = 1) -> list[int]:
        """Acquire ``n`` slots for sequences that start together."""
        got = []
        try:
            for _ in range(n):
                got.append(self.cache.acquire())
        except CacheError:
            for s in got:
                self.cache.release(s)
            raise
        return got

    def close(self, slots) -> None:
        """Give slots (and what they hold) back."""
        for s in slots:
            self.cache.release(s)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, length: int) -> None:
        """Keep the first ``length`` positions of a slot (to continue from a shared prefix)."""
        self.cache.truncate(slot, length)

    def mark(self):
        """A point on the device's timeline (a CUDA event on the current stream); two of them give the
        device time of what was queued between them (``elapsed_ms``).  The generation loop marks every
        step this way."""
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    @staticmethod
    def elapsed_ms(a, b) -> float:
        b.synchronize()
        return a.elapsed_time(b)

    def memory_report(self) -> dict:
        """Bytes held on the device: weights, cache, scratch."""
        seen, weights = set(), 0
        def add(t):
            nonlocal weights
            if isinstance(t, torch.Tensor) and t.is_cuda and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                weights += t.numel() * t.element_size()
        for part in self.model.all_parts():
            for v in vars(part).values():
                add(v)
        return {"weights": weights, "cache": self.cache.nbytes(), "scratch": self.rt.arena._buf.numel(),
                "cache_positions": self.max_tokens, "slots": self.cache.n_slots}

    # ---- the step ----------------------------------------------------------------------
    def step(self, slots, tokens, want=None, borrow: bool = False) -> torch.Tensor:
        """slots[i] continues with tokens[i]; want[i] lists the places among tokens[i] whose
        logits are asked for (None: the last of each).  Returns float32 [sum(len(want[i])),
        vocabulary] on the device, in the order of the entries and of ``want``.
        ``borrow``: the caller reads the result before the next step and needs no copy of its own
        (a captured decode step writes its logits to the same memory every time)."""
        self._borrow = borrow
        B = len(slots)
        if len(tokens) != B:
            raise StepError("step: one token list for each slot is needed")
        if want is None and B and all(len(t) == 1 for t in tokens):
            return self._step_one_token_each(slots, tokens)
        if want is None:
            want = [[len(t) - 1] if len(t) else [] for t in tokens]
        if len(want) != B:
            raise StepError("step: one list of wanted places for each slot is needed")
        if len(set(slots)) != B:
            raise StepError("step: a slot is named twice")
        V = self.spec.vocab_size
        lens_after = {}
        for s, t, w in zip(slots, tokens, want):
            self._check_slot(s)
            if len(t) == 0:
                if len(w):
                    raise StepError("step: logits wanted of a sequence that brings no token")
                continue
            a = np.asarray(t)
            if a.ndim != 1 or not np.issubdtype(a.dtype, np.integer):
                raise StepError("step: tokens must be flat lists of integers")
            if a.min() < 0 or a.max() >= V:
                bad = int(a[(a < 0) | (a >= V)][0])
                raise StepError(f"step: token id {bad} is outside the vocabulary [0, {V})")
            for p in w:
                if not (0 <= p < len(t)):
                    raise StepError(f"step: wanted place {p} is outside the {len(t)} tokens given")
            n_after = self.cache.length(s) + len(t)
            if n_after > self.max_context:
                raise StepError(f"step: slot {s} would reach {n_after} positions; the limit is "
                                f"{self.max_context}")
            lens_after[s] = n_after
        try:
            self.cache.can_hold(lens_after)
        except CacheError as e:
            raise StepError(str(e)) from e

        # rows of the result: entry by entry, in the order of ``want``
        n_want = sum(len(w) for w in want)
        row_of = {}
        r = 0
        for i, w in enumerate(want):
            for p in w:
                row_of.setdefault((i, p), []).append(r)
                r += 1
        done = [0] * B
        pieces, piece_rows = [], []
        while True:
            budget = self.max_step_tokens
            sel, new, before, wrows, wdst = [], [], [], [], []
            base = 0
            for i in range(B):
                left = len(tokens[i]) - done[i]
                if left <= 0 or budget <= 0:
                    continue
                n = min(left, self.seq_chunk, budget)
                budget -= n
                sel.append(i)
                new.append(tokens[i][done[i]:done[i] + n])
                before.append(self.cache.length(slots[i]))
                for j in range(n):
                    for dst in row_of.get((i, done[i] + j), ()):
                        wrows.append(base + j)
                        wdst.append(dst)
                base += n
            if not sel:
                break
            pieces.append(self._pass([slots[i] for i in sel], new, before, wrows))
            piece_rows.append(wdst)
            for i, t in zip(sel, new):
                done[i] += len(t)
        if not pieces:
            return torch.empty((0, V), dtype=torch.float32, device=self.device)
        order = [d for rows in piece_rows for d in rows]
        if order == list(range(n_want)):
            return pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
        out = torch.empty((n_want, V), dtype=torch.float32, device=self.device)
        out[torch.tensor(order, dtype=torch.long, device=self.device)] = torch.cat(pieces, dim=0)
        return out

    def _check_slot(self, s) -> None:
        try:
            self.cache.slots.check(s)
        except CacheError as e:
            raise StepError(f"step: {e}") from e

    def _step_one_token_each(self, slots, tokens) -> torch.Tensor:
        """The common decode step, checked with less work: one token a sequence, every logit wanted."""
        B = len(slots)
        if len(set(slots)) != B:
            raise StepError("step: a slot is named twice")
        V = self.spec.vocab_size
        ids = [t[0] for t in tokens]
        if min(ids) < 0 or max(ids) >= V:
            bad = [i for i in ids if i < 0 or i >= V][0]
            raise StepError(f"step: token id {bad} is outside the vocabulary [0, {V})")
        before, after = [], {}
        for s in slots:
            self._check_slot(s)
            n = self.cache.slots.length[s]
            if n + 1 > self.max_context:
                raise StepError(f"step: slot {s} would reach {n + 1} positions; the limit is {self.max_context}")
            before.append(n)
            if n % PAGE == 0:                    # only a sequence at a page's edge needs a new page
                after[s] = n + 1
        if after:
            try:
                self.cache.can_hold(after)
            except CacheError as e:
                raise StepError(str(e)) from e
        return self._pass(slots, tokens, before, list(range(B)))

    @property
    def feeds_from_device(self) -> bool:
        """Whether ``step_fed`` is there: decode steps are replayed graphs that read a record on the device."""
        return bool(self.use_graphs)

    def step_fed(self, slots, ids_dev: torch.Tensor) -> torch.Tensor:
        """The common decode step with the token ids already on the device (int32, one a slot, for
        instance where the sampler has just put them): the step can be queued before the host has
        seen the ids, so the device never waits for the host between two steps.  An id outside the
        vocabulary raises the status flag that ``check_errors`` reports.  The logits returned are
        the graph's own buffer: they hold until the next step with as many sequences."""
        if not self.feeds_from_device:
            raise StepError("step_fed: this engine does not replay captured decode steps")
        B = len(slots)
        if len(set(slots)) != B:
            raise StepError("step: a slot is named twice")
        if ids_dev.dtype != torch.int32 or ids_dev.device != self.device or ids_dev.numel() < B:
            raise StepError("step_fed: token ids must be int32 on the engine's device, one a slot")
        before, after = [], {}
        for s in slots:
            self._check_slot(s)
            n = self.cache.slots.length[s]
            if n + 1 > self.max_context:
                raise StepError(f"step: slot {s} would reach {n + 1} positions; the limit is {self.max_context}")
            before.append(n)
            if n % PAGE == 0:
                after[s] = n + 1
        if after:
            try:
                self.cache.can_hold(after)
            except CacheError as e:
                raise StepError(str(e)) from e
        self._borrow = True
        try:
            return self._pass(slots, [[0]] * B, before, list(range(B)), ids_dev=ids_dev)
        finally:
            self._borrow = False

    def _pass(self, slots, new_tokens, before, want_rows, ids_dev=None) -> torch.Tensor:
        """One pass through the layers: reserve pages, lay the batch out, run, commit."""
        for s, t, b in zip(slots, new_tokens, before):
            self.cache.reserve(s, b + len(t))
        B = len(slots)
        tables = self.cache.tables(slots)
        decode = self.use_graphs and all(len(t) == 1 for t in new_tokens) and list(want_rows) == list(range(B))
        if decode:
            logits = self._decode_pass(slots, new_tokens, before, want_rows, tables, ids_dev)
        else:
            batch = build_step_batch(slots, new_tokens, before, want_rows, tables, self.device, self._ring)
            self.last_h2d_bytes = batch.host["n_ints"] * 4
            logits = self.model.forward(batch, self.cache)
        for s, t in zip(slots, new_tokens):
            self.cache.commit(s, len(t))
        return logits

    def _decode_key(self, B: int, longest: int):
        """What a captured decode step depends on besides the record it reads: the number of
        sequences and, through the slices of the key range, the length of the longest one."""
        from ..kernels import attn_tc
        key = [B]
        for g in self.cache.kv_groups:
            key.append(attn_tc.decode_slices(B, g.need.n_kv_heads, longest, g.need.window))
        return tuple(key)

    def _decode_pass(self, slots, new_tokens, before, want_rows, tables, ids_dev=None) -> torch.Tensor:
        B = len(slots)
        longest = max(before) + 1
        key = self._decode_key(B, longest)
        ids = [t[0] for t in new_tokens]
        entry = self._graphs.get(key)
        if entry is None:
            # The first step of this shape runs the ordinary way (which also loads libraries, makes
            # tensor maps and sizes the scratch) and its logits are the step's result; the capture
            # that follows records the same launches without running them, so the step has been
            # executed once: a part that keeps state of its own advances it once, not twice.
            record = DecodeRecord(B, [t.shape[1] for t in tables], self.device, self._ring)
            batch = record.update(slots, ids, before, tables, ids_dev)
            self.last_h2d_bytes = record.total * 4
            first = self.model.forward(batch, self.cache)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            l0 = self.rt.launches
            with torch.cuda.graph(graph):
                logits = self.model.forward(batch, self.cache)
            self._graphs[key] = (graph, record, logits, self.rt.launches - l0)
            self.rt.launches = l0
            return first
        graph, record, logits, n_launch = entry
        record.update(slots, ids, before, tables, ids_dev)
        self.last_h2d_bytes = record.total * 4
        graph.replay()
        self.rt.launches += n_launch
        return logits if getattr(self, "_borrow", False) else logits.clone()
