"""Running the sampling kernel for a batch: one record of parameters a row, the recent
tokens of the rows that use penalties, one token id back for each row."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def stream_seed(seed: int, sequence: int) -> int:
    """The key of one sequence's random stream: it depends on the request's seed and on the
    sequence's index among the requests, never on the batch the sequence runs in."""
    return _mix64((seed & _MASK) ^ _mix64(sequence + 1))


def uniform_of(stream: int, counter: int) -> float:
    """The uniform number in [0, 1) that the kernel draws for this stream and counter."""
    r = _mix64(stream ^ _mix64((counter + 0x632BE59BD9B4E019) & _MASK))
    return float(np.float32(r >> 40) * np.float32(1.0 / 16777216.0))


class Sampler:
    """``runtime`` (optional): the engine's runtime; its status flags then come back with the token
    ids in the same copy, and a raised flag is an error here.

    The recent tokens that penalties look back on live in rings on the device, one a random stream
    (a sequence): the first call for a stream sends the end of its history, after that the kernel
    appends each token it samples and the host sends nothing.  The host only checks that the
    history it is given has grown by exactly the tokens sampled here; anything else (a new
    sequence under an old stream number, an edited history) is sent afresh."""

    RINGS = 4096               # streams whose rings are held at once

    def __init__(self, device, vocab_size: int, runtime=None):
        self.device, self.vocab_size = torch.device(device), int(vocab_size)
        self.rt = runtime
        self._work = None
        self._cache_key = None
        self._cache = None
        if runtime is not None and getattr(runtime, "status_and_ids", None) is not None:
            self._out = runtime.status_and_ids
        else:
            self._out = torch.zeros(4 + 4096, dtype=torch.int32, device=self.device)
        self._dummy_i = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._dummy_f = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._hist = None          # [RINGS, capacity] int32
        self._hist_len = None      # [RINGS] int32: tokens put into each ring so far
        self._ring_of: dict = {}   # (stream, row of that stream) -> (ring, length of the history it mirrors, last token)
        self._free_rings: list = []
        self._last = None          # rows of the call before: (identity, rings, keys)
        self._landing = [None, None]   # pinned host buffers the ids are copied into, used in turn
        self._turn = 0
        self._keys = []

    # ---- rings of recent tokens ------------------------------------------------------------
    def _ensure_rings(self, window: int) -> None:
        cap = max(64, -(-window // 64) * 64)
        if self._hist is None or self._hist.shape[1] < cap:
            self._hist = torch.zeros((self.RINGS, cap), dtype=torch.int32, device=self.device)
            self._hist_len = torch.zeros(self.RINGS, dtype=torch.int32, device=self.device)
            self._ring_of.clear()
            self._free_rings = list(range(self.RINGS))[::-1]
            self._cache_key = None

    def _rings_for(self, params: list, streams: list, recents: list, counters: list) -> list:
        """Ring numbers for the rows that use history (-1 for the others).  A ring is (re)filled from
        ``recents`` when its stream is new or draws its first token, or when the history given is
        not the one the ring mirrors plus the token that was sampled into it last."""
        window = max(p.history_window() for p in params)
        self._ensure_rings(window)
        cap = self._hist.shape[1]
        rings, fresh = [], []
        self._keys = keys = []                 # a ring belongs to (stream, which row of that stream in the call)
        times: dict = {}
        for i, p in enumerate(params):
            k = times.get(streams[i], 0)
            times[streams[i]] = k + 1
            keys.append((streams[i], k))
            if p.history_window() <= 0:
                rings.append(-1)
                continue
            hist = recents[i] if recents is not None else ()
            known = self._ring_of.get(keys[i])
            if known is None:
                if not self._free_rings:          # every ring taken: start over (rows in use are refilled below)
                    self._ring_of.clear()
                    self._free_rings = list(range(self.RINGS))[::-1]
                    self._cache_key = None
                    return self._rings_for(params, streams, recents, counters)
                known = (self._free_rings.pop(), -1, -1)
            ring, length, last = known
            if counters[i] == 0 or length != len(hist) or (length > 0 and hist[-1] != last):
                fresh.append((ring, list(hist[-cap:])))
            self._ring_of[keys[i]] = (ring, len(hist), -1)
            rings.append(ring)
        if fresh:
            flat = np.zeros((len(fresh), cap), dtype=np.int32)
            lens = np.zeros(len(fresh), dtype=np.int32)
            for j, (_, tail) in enumerate(fresh):
                flat[j, :len(tail)] = tail
                lens[j] = len(tail)
            idx = torch.tensor([r for r, _ in fresh], dtype=torch.long, device=self.device)
            self._hist.index_copy_(0, idx, torch.from_numpy(flat).to(self.device))
            self._hist_len.index_copy_(0, idx, torch.from_numpy(lens).to(self.device))
        return rings

    def forget(self, streams) -> None:
        """Give back the rings of streams that have ended (optional: rings are recycled anyway)."""
        gone = set(streams)
        for key in [k for k in self._ring_of if k[0] in gone]:
            self._free_rings.append(self._ring_of.pop(key)[0])

    def _records(self, params: list, streams: list, rings: tuple):
        """The per-row records for these parameters, streams and rings, without counters (kept on the
        device from call to call: a batch samples with the same parameters every step)."""
        key = (tuple(map(id, params)), tuple(streams), rings)
        if key != self._cache_key:
            rec = np.zeros(len(params), dtype=ops.SAMPLE_DTYPE)
            bias_ids, bias_vals = [], []
            for i, p in enumerate(params):
                r = rec[i]
                r["temperature"], r["top_p"], r["min_p"], r["rep_penalty"] = p.temperature, p.top_p, p.min_p, p.rep_penalty
                r["freq_penalty"], r["presence_penalty"] = p.frequency_penalty, p.presence_penalty
                r["dry_multiplier"], r["dry_base"] = p.dry_multiplier, p.dry_base
                r["top_k"], r["repeat_last_n"], r["dry_last_n"] = p.top_k, p.repeat_last_n, p.dry_last_n
                r["dry_allowed_len"] = p.dry_allowed_len
                r["seed"] = streams[i] & _MASK
                if rings[i] >= 0:
                    r["n_recent"], r["recent_offset"] = -1, rings[i]
                r["n_bias"], r["bias_offset"] = len(p.logit_bias), len(bias_ids)
                for k, v in p.logit_bias.items():
                    bias_ids.append(int(k))
                    bias_vals.append(float(v))
            plain = all(g < 0 for g in rings) and not bias_ids
            greedy = all(p.greedy for p in params)
            dev = torch.from_numpy(rec.view(np.uint8).reshape(-1).copy()).to(self.device)
            bid = bval = None
            if bias_ids:
                bid = torch.tensor(bias_ids, dtype=torch.int32, device=self.device)
                bval = torch.tensor(bias_vals, dtype=torch.float32, device=self.device)
            # the parameter objects are kept so that their ids in the key stay theirs
            self._cache_key, self._cache = key, (rec, plain, greedy, dev, bid, bval, list(params))
        return self._cache

    def sample(self, logits: torch.Tensor, params: list, streams: list, counters: list,
               recents: list | None = None) -> list[int]:
        """logits: float32 [n, vocab] on the device; params[i], streams[i] (from stream_seed),
        counters[i] (tokens drawn so far), recents[i] (the sequence's tokens so far: what penalties
        look back on) for row i."""
        return self.begin(logits, params, streams, counters, recents).wait()

    def begin(self, logits: torch.Tensor, params: list, streams: list, counters: list,
              recents: list | None = None, continuing: bool = False) -> "Pending":
        """The same without waiting: the kernel is launched, the ids start on their way to the host,
        and ``wait()`` of what is returned gives them.  ``ids_dev`` of it holds them on the device
        (until the next call) for a step that is queued before the host has seen them.
        ``continuing``: these are the rows of the call before, one token later; the rings of recent
        tokens are taken as the kernel left them and ``recents`` is not looked at."""
        n = logits.shape[0]
        if n > self._out.numel() - 4:
            raise ValueError(f"at most {self._out.numel() - 4} rows a call")
        if n == 0:
            return Pending(self, 0, None, None, (), ())
        dev = self.device
        uses = any(p.history_window() > 0 for p in params)
        if continuing:
            if self._last is None or self._last[0] != (tuple(map(id, params)), tuple(streams)):
                raise ValueError("continuing: not the rows of the call before")
            rings, keys = self._last[1], self._last[2]
        else:
            rings = tuple(self._rings_for(params, streams, recents, counters)) if uses else (-1,) * n
            keys = tuple(self._keys) if uses else ()
        self._last = ((tuple(map(id, params)), tuple(streams)), rings, keys)
        base, plain, greedy, base_dev, bid_dev, bval_dev, _ = self._records(params, streams, rings)
        if all(c == counters[0] for c in counters):
            # rows that have drawn equally often: the records stay, the count is an argument
            params_dev, counter_add = base_dev, int(counters[0])
        else:
            rec = base.copy()
            rec["counter"] = np.asarray(counters, dtype=np.uint64)
            params_dev, counter_add = torch.from_numpy(rec.view(np.uint8).reshape(-1)).to(dev, non_blocking=True), 0
        work = None
        if not plain:
            if self._work is None or self._work.numel() < n * self.vocab_size:
                self._work = torch.empty(n * self.vocab_size, dtype=torch.float32, device=dev)
            work = self._work
        out = self._out[4:4 + n]
        ops.sample(logits, work, params_dev, self._dummy_i, bid_dev if bid_dev is not None else self._dummy_i,
                   bval_dev if bval_dev is not None else self._dummy_f, out, counter_add,
                   self._hist if uses else None, self._hist_len if uses else None)
        # the status flags travel with the ids; two landing places, so that a call may begin before
        # the one before it has been waited for
        self._turn ^= 1
        if self._landing[self._turn] is None:
            self._landing[self._turn] = torch.empty(self._out.numel(), dtype=torch.int32, pin_memory=True)
        pin = self._landing[self._turn]
        pin[:4 + n].copy_(self._out[:4 + n], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return Pending(self, n, pin, done, rings if uses else (), keys)


class Pending:
    """Token ids on their way from the device."""

    def __init__(self, sampler, n, pin, done, rings, keys):
        self.sampler, self.n, self.pin, self.done, self.rings, self.keys = sampler, n, pin, done, rings, keys
        self.ids_dev = sampler._out[4:4 + n] if n else None

    def wait(self) -> list[int]:
        if self.n == 0:
            return []
        self.done.synchronize()
        host = self.pin[:4 + self.n].tolist()
        smp = self.sampler
        if smp.rt is not None and any(host[:4]):
            smp.rt.check_status()
        ids = host[4:]
        for i, g in enumerate(self.rings):     # what each ring now holds: its history plus the token just drawn
            if g >= 0:
                known = smp._ring_of.get(self.keys[i])
                if known is not None and known[0] == g:
                    smp._ring_of[self.keys[i]] = (g, known[1] + 1, ids[i])
        return ids
