"""Running the sampling kernel for a batch: one record of parameters a row, the recent
tokens of the rows that use penalties, one token id back for each row."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams

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
    ids in the same copy, and a raised flag is an error here."""

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

    def _records(self, params: list, streams: list):
        """The per-row records for these parameters and streams, without counters and history
        (kept from call to call: a batch samples with the same parameters every step)."""
        key = (tuple((id(p), p.temperature, p.top_k, p.top_p, p.min_p, p.rep_penalty, p.repeat_last_n,
                      p.frequency_penalty, p.presence_penalty, p.dry_multiplier, p.dry_last_n, len(p.logit_bias))
                     for p in params), tuple(streams))
        if key != self._cache_key:
            rec = np.zeros(len(params), dtype=ops.SAMPLE_DTYPE)
            plain = True
            for i, p in enumerate(params):
                r = rec[i]
                r["temperature"], r["top_p"], r["min_p"], r["rep_penalty"] = p.temperature, p.top_p, p.min_p, p.rep_penalty
                r["freq_penalty"], r["presence_penalty"] = p.frequency_penalty, p.presence_penalty
                r["dry_multiplier"], r["dry_base"] = p.dry_multiplier, p.dry_base
                r["top_k"], r["repeat_last_n"], r["dry_last_n"] = p.top_k, p.repeat_last_n, p.dry_last_n
                r["dry_allowed_len"] = p.dry_allowed_len
                r["seed"] = streams[i] & _MASK
                if p.history_window() > 0 or p.logit_bias:
                    plain = False
            greedy = all(p.greedy for p in params)
            dev = None
            if plain:          # nothing changes from step to step but the counters: keep the records on the device
                dev = torch.from_numpy(rec.view(np.uint8).reshape(-1).copy()).to(self.device)
            self._cache_key, self._cache = key, (rec, plain, greedy, dev)
        return self._cache

    def sample(self, logits: torch.Tensor, params: list, streams: list, counters: list,
               recents: list | None = None) -> list[int]:
        """logits: float32 [n, vocab] on the device; params[i], streams[i] (from stream_seed),
        counters[i] (tokens drawn so far), recents[i] (tokens generated so far) for row i."""
        n = logits.shape[0]
        if n == 0:
            return []
        if n > self._out.numel() - 4:
            raise ValueError(f"at most {self._out.numel() - 4} rows a call")
        base, plain, greedy, base_dev = self._records(params, streams)
        dev = self.device
        same = plain and all(c == counters[0] for c in counters)
        rec = None
        if not same:
            rec = base.copy()
            rec["counter"] = np.asarray(counters, dtype=np.uint64)
        recent_dev, bid_dev, bval_dev = self._dummy_i, self._dummy_i, self._dummy_f
        if not plain:
            recent_flat, bias_ids, bias_vals = [], [], []
            for i, p in enumerate(params):
                win = p.history_window()
                hist = list(recents[i][-win:]) if (recents is not None and win > 0) else []
                rec[i]["n_recent"], rec[i]["recent_offset"] = len(hist), len(recent_flat)
                recent_flat.extend(hist)
                rec[i]["n_bias"], rec[i]["bias_offset"] = len(p.logit_bias), len(bias_ids)
                for k, v in p.logit_bias.items():
                    bias_ids.append(int(k))
                    bias_vals.append(float(v))
            if recent_flat:
                recent_dev = torch.tensor(recent_flat, dtype=torch.int32).to(dev, non_blocking=True)
            if bias_ids:
                bid_dev = torch.tensor(bias_ids, dtype=torch.int32).to(dev, non_blocking=True)
                bval_dev = torch.tensor(bias_vals, dtype=torch.float32).to(dev, non_blocking=True)
        if same:               # rows that have drawn equally often: the records stay, the count is an argument
            params_dev, counter_add = base_dev, int(counters[0])
        else:
            params_dev, counter_add = torch.from_numpy(rec.view(np.uint8).reshape(-1)).to(dev, non_blocking=True), 0
        work = None
        if not (greedy and plain):
            if self._work is None or self._work.numel() < n * self.vocab_size:
                self._work = torch.empty(n * self.vocab_size, dtype=torch.float32, device=dev)
            work = self._work
        out = self._out[4:4 + n]
        ops.sample(logits, work, params_dev, recent_dev, bid_dev, bval_dev, out, counter_add)
        host = self._out[:4 + n].cpu().tolist()          # the status flags travel with the ids
        if self.rt is not None and any(host[:4]):
            self.rt.check_status()
        return host[4:]
