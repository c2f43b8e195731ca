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
    def __init__(self, device, vocab_size: int):
        self.device, self.vocab_size = torch.device(device), int(vocab_size)
        self._work = None

    def sample(self, logits: torch.Tensor, params: list, streams: list, counters: list,
               recents: list | None = None) -> list[int]:
        """logits: float32 [n, vocab] on the device; params[i], streams[i] (from stream_seed),
        counters[i] (tokens drawn so far), recents[i] (tokens generated so far) for row i."""
        n = logits.shape[0]
        if n == 0:
            return []
        rec = np.zeros(n, dtype=ops.SAMPLE_DTYPE)
        recent_flat, bias_ids, bias_vals = [], [], []
        need_work = False
        for i, p in enumerate(params):
            r = rec[i]
            r["temperature"], r["top_p"], r["min_p"], r["rep_penalty"] = p.temperature, p.top_p, p.min_p, p.rep_penalty
            r["freq_penalty"], r["presence_penalty"] = p.frequency_penalty, p.presence_penalty
            r["dry_multiplier"], r["dry_base"] = p.dry_multiplier, p.dry_base
            r["top_k"], r["repeat_last_n"], r["dry_last_n"] = p.top_k, p.repeat_last_n, p.dry_last_n
            r["dry_allowed_len"] = p.dry_allowed_len
            r["seed"], r["counter"] = streams[i] & _MASK, counters[i]
            win = p.history_window()
            hist = list(recents[i][-win:]) if (recents is not None and win > 0) else []
            r["n_recent"], r["recent_offset"] = len(hist), len(recent_flat)
            recent_flat.extend(hist)
            r["n_bias"], r["bias_offset"] = len(p.logit_bias), len(bias_ids)
            for k, v in p.logit_bias.items():
                bias_ids.append(int(k))
                bias_vals.append(float(v))
            if not p.greedy or hist or p.logit_bias:
                need_work = True
        dev = self.device
        params_dev = torch.from_numpy(rec.view(np.uint8).reshape(-1)).to(dev, non_blocking=True)
        recent_dev = torch.tensor(recent_flat or [0], dtype=torch.int32).to(dev, non_blocking=True)
        bid_dev = torch.tensor(bias_ids or [0], dtype=torch.int32).to(dev, non_blocking=True)
        bval_dev = torch.tensor(bias_vals or [0.0], dtype=torch.float32).to(dev, non_blocking=True)
        work = None
        if need_work:
            if self._work is None or self._work.numel() < n * self.vocab_size:
                self._work = torch.empty(n * self.vocab_size, dtype=torch.float32, device=dev)
            work = self._work
        out = torch.empty(n, dtype=torch.int32, device=dev)
        ops.sample(logits, work, params_dev, recent_dev, bid_dev, bval_dev, out)
        return out.cpu().tolist()
