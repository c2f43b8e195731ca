"""Storage of the cache on the device and its views for one step.

Runs of the model's run list are grouped by what they need.  A group of runs that keep keys
and values of the same shape and the same window shares one pool of pages of 64 positions:
K and V of shape [runs, pages, kv heads, 64, head size].  A sequence holds a list of pages
in every group; a group with a window holds only as many pages as the window (plus the
longest run of new tokens in a step) needs and wraps around, position p lying at p modulo
that span.  Runs with fixed-size state get one array [runs, slots, ...] a group, zeroed
when a slot is acquired.

The reference allocates [kv heads, context, head size] for every slot and layer
(src/kv_cache/kv_cache.cpp:35-72), masks the window over the same buffers
(src/model/qwen_block.cpp:742-745) and keeps recurrent state in an array of its own beside
the KV cache, indexed densely over the layers that need it (src/kv_cache/recurrent_state.cpp:
35-49, reset at a sequence's start :96-106).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .book import PAGE, CacheError, PageAllocator, SlotBook


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class KVView:
    """What an attention kernel needs to reach one run's keys and values in this step."""
    k: torch.Tensor            # [pages, kv heads, PAGE, head size]
    v: torch.Tensor
    table: torch.Tensor        # int32 [sequences of the step, pages a sequence]
    ring: int                  # positions a sequence's pages span
    page: int
    window: Optional[int]
    owner: bool                # False: this run reads another run's cache and must not write


@dataclass
class RunCache:
    kv: Optional[KVView] = None
    state: Optional[torch.Tensor] = None     # [slots, ...]; rows are slot numbers
    owner: bool = True


class KVGroup:
    def __init__(self, need: KVNeed, runs: list, n_pages: int, ring_pages: int, pages_per_seq: int,
                 n_slots: int, dtype, device, poison: bool):
        self.need, self.runs = need, list(runs)
        self.index = {r: i for i, r in enumerate(self.runs)}
        self.n_pages, self.ring_pages, self.pages_per_seq = n_pages, ring_pages, pages_per_seq
        self.pool = PageAllocator(n_pages)
        self.pages_of = [[] for _ in range(n_slots)]
        shape = (len(self.runs), n_pages, need.n_kv_heads, PAGE, need.head_dim)
        self.k = torch.empty(shape, dtype=dtype, device=device)
        self.v = torch.empty(shape, dtype=dtype, device=device)
        if poison:
            self.k.fill_(float("nan"))
            self.v.fill_(float("nan"))

    def pages_needed(self, length: int) -> int:
        return min(_ceil_div(length, PAGE), self.ring_pages)

    @property
    def ring(self) -> int:
        return self.ring_pages * PAGE

    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class StateGroup:
    def __init__(self, need: StateNeed, runs: list, n_slots: int, device):
        self.need, self.runs = need, list(runs)
        self.index = {r: i for i, r in enumerate(self.runs)}
        dt = getattr(torch, need.dtype)
        self.data = torch.zeros((len(self.runs), n_slots) + tuple(need.shape), dtype=dt, device=device)


class Cache:
    """Slots, pages and state for one model on one device.

    needs:        for each run of the run list: None, KVNeed, StateNeed or a tuple of them
    cache_from:   for each run: None or the index of the run whose cache it reads
    max_tokens:   positions that live sequences may hold together (each rounded up to a page)
    max_context:  positions one sequence may reach
    step_chunk:   the most new tokens a sequence brings in one step (sizes a window's span)
    """

    def __init__(self, needs, cache_from, max_tokens: int, max_context: int, n_slots: int,
                 step_chunk: int, dtype=torch.float32, device="cpu", poison: bool = False):
        self.n_slots, self.max_context, self.step_chunk = int(n_slots), int(max_context), int(step_chunk)
        self.max_tokens = int(max_tokens)
        self.slots = SlotBook(n_slots)
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self._kv_of_run: dict[int, KVGroup] = {}
        self._state_of_run: dict[int, StateGroup] = {}
        self.cache_from = list(cache_from)
        total_pages = _ceil_div(self.max_tokens, PAGE)
        ctx_pages = _ceil_div(self.max_context, PAGE)
        kv_runs: dict[KVNeed, list] = {}
        st_runs: dict[StateNeed, list] = {}
        for r, need in enumerate(needs):
            if self.cache_from[r] is not None:
                src = self.cache_from[r]
                if not (0 <= src < r) or self.cache_from[src] is not None:
                    raise CacheError(f"run {r} reads the cache of run {src}, which must be an "
                                     f"earlier run with a cache of its own")
                continue
            for n in (need if isinstance(need, tuple) else (need,)):
                if isinstance(n, KVNeed):
                    kv_runs.setdefault(n, []).append(r)
                elif isinstance(n, StateNeed):
                    st_runs.setdefault(n, []).append(r)
                elif n is not None:
                    raise CacheError(f"run {r}: unknown cache need {n!r}")
        for need, runs in kv_runs.items():
            if need.window is None:
                ring_pages = ctx_pages
            else:
                ring_pages = min(ctx_pages, _ceil_div(need.window + self.step_chunk - 1, PAGE))
            n_pages = min(total_pages, self.n_slots * ring_pages)
            g = KVGroup(need, runs, n_pages, ring_pages, ring_pages, self.n_slots, dtype, device, poison)
            self.kv_groups.append(g)
            for r in runs:
                self._kv_of_run[r] = g
        for need, runs in st_runs.items():
            g = StateGroup(need, runs, self.n_slots, device)
            self.state_groups.append(g)
            for r in runs:
                self._state_of_run[r] = g

    # ---- slots ---------------------------------------------------------------------------
    def acquire(self) -> int:
        s = self.slots.acquire()
        for g in self.state_groups:
            g.data[:, s].zero_()
        return s

    def release(self, slot: int) -> None:
        self.slots.check(slot)
        for g in self.kv_groups:
            g.pool.give_back(g.pages_of[slot])
            g.pages_of[slot] = []
        self.slots.release(slot)

    def length(self, slot: int) -> int:
        self.slots.check(slot)
        return self.slots.length[slot]

    def can_hold(self, lengths_after: dict) -> None:
        """Raise unless every slot of ``lengths_after`` (slot -> length) can grow to that length."""
        for g in self.kv_groups:
            extra = 0
            for s, n in lengths_after.items():
                extra += max(0, g.pages_needed(n) - len(g.pages_of[s]))
            if extra > g.pool.n_free:
                raise CacheError(f"cache is full: the step needs {extra} more pages of {PAGE} "
                                 f"positions, {g.pool.n_free} of {g.n_pages} are free "
                                 f"(max_tokens={self.max_tokens})")

    def reserve(self, slot: int, length_after: int) -> None:
        self.slots.check(slot)
        if length_after > self.max_context:
            raise CacheError(f"sequence in slot {slot} would reach {length_after} positions; "
                             f"the limit is {self.max_context}")
        for g in self.kv_groups:
            more = g.pages_needed(length_after) - len(g.pages_of[slot])
            if more > 0:
                g.pages_of[slot].extend(g.pool.take(more))

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions from ``length`` on (prefix reuse: the reference truncates a slot to
        the common prefix of its tokens and a new prompt, src/kv_cache/kv_cache.cpp:141-157).  A
        sequence with windowed or state-carrying runs cannot go back (the reference forbids it for
        its recurrent models, include/ultima/model/imodel.hpp:193-202), except to its start."""
        self.slots.check(slot)
        if not (0 <= length <= self.slots.length[slot]):
            raise CacheError(f"cannot truncate slot {slot} of length {self.slots.length[slot]} to {length}")
        if length > 0 and (self.state_groups or any(g.need.window is not None for g in self.kv_groups)):
            raise CacheError("a sequence with a window or with state can only be truncated to its start")
        for g in self.kv_groups:
            keep = g.pages_needed(length)
            g.pool.give_back(g.pages_of[slot][keep:])
            del g.pages_of[slot][keep:]
        if length == 0:
            for g in self.state_groups:
                g.data[:, slot].zero_()
        self.slots.length[slot] = length

    def commit(self, slot: int, n_new: int) -> None:
        self.slots.check(slot)
        self.slots.length[slot] += n_new

    # ---- views for a step ------------------------------------------------------------------
    def tables(self, slots: list) -> list:
        """For each KV group an int32 array [len(slots), pages a sequence] (unused entries 0)."""
        out = []
        for g in self.kv_groups:
            t = np.zeros((len(slots), g.pages_per_seq), dtype=np.int32)
            for i, s in enumerate(slots):
                p = g.pages_of[s]
                t[i, :len(p)] = p
            out.append(t)
        return out

    def run_cache(self, run: int, tables_dev: list) -> RunCache:
        """The view of run ``run``; ``tables_dev`` are this step's tables on the device, in
        the order of ``kv_groups``."""
        src = self.cache_from[run]
        owner = src is None
        r = run if owner else src
        out = RunCache(owner=owner)
        g = self._kv_of_run.get(r)
        if g is not None:
            i = g.index[r]
            out.kv = KVView(g.k[i], g.v[i], tables_dev[self.kv_groups.index(g)], g.ring, PAGE,
                            g.need.window, owner)
        sg = self._state_of_run.get(r)
        if sg is not None:
            out.state = sg.data[sg.index[r]]
        return out

    def nbytes(self) -> int:
        return sum(g.nbytes() for g in self.kv_groups) + \
            sum(g.data.numel() * g.data.element_size() for g in self.state_groups)

    def pages_held(self) -> int:
        return sum(len(p) for g in self.kv_groups for p in g.pages_of)
