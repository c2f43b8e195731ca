"""One step's worth of tokens, laid out for the kernels.

A step brings, for each of its sequences, some new tokens that follow what the sequence's
slot already holds.  Tokens of all sequences are packed one after another; for every token
the kernels get its id, its absolute position and the index of its sequence in the step,
and for every sequence its first row, its length before the step and its slot.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    tok_ids: torch.Tensor         # int32 [T]
    tok_pos: torch.Tensor         # int32 [T]  absolute position of each token
    tok_seq: torch.Tensor         # int32 [T]  index of the token's sequence in this step
    seq_start: torch.Tensor       # int32 [B + 1] first row of each sequence
    seq_before: torch.Tensor      # int32 [B] positions held before this step
    seq_slot: torch.Tensor        # int32 [B]
    want_rows: torch.Tensor       # int32 [W] rows whose logits are asked for
    tables: list                  # per KV group: int32 [B, pages a sequence]
    max_new: int = 0              # longest run of new tokens of a sequence
    max_after: int = 0            # longest sequence after the step
    host: dict = field(default_factory=dict)


def build_step_batch(slots, new_tokens, before, want_rows, tables_np, device, pin=None) -> StepBatch:
    """slots: slot of each sequence; new_tokens: list of int sequences; before: positions
    already held; want_rows: rows (in the packed order) whose logits are wanted;
    tables_np: per KV group an int32 array [B, pages]."""
    B = len(slots)
    lens = np.fromiter((len(t) for t in new_tokens), dtype=np.int64, count=B)
    T = int(lens.sum())
    start = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(lens, out=start[1:])
    ids = np.concatenate([np.asarray(t, dtype=np.int32) for t in new_tokens]) if T else np.zeros(0, np.int32)
    seq = np.repeat(np.arange(B, dtype=np.int32), lens)
    before = np.asarray(before, dtype=np.int32)
    pos = (np.arange(T, dtype=np.int32) - start[:-1][seq] + before[seq]).astype(np.int32)
    want = np.asarray(want_rows, dtype=np.int32)
    parts = [ids, pos, seq, start, before, np.asarray(slots, dtype=np.int32), want] + \
        [t.reshape(-1) for t in tables_np]
    sizes = [p.size for p in parts]
    # every part starts on a 16-byte boundary of one buffer, moved in one copy
    offs, o = [], 0
    for s in sizes:
        offs.append(o)
        o += -(-s // 4) * 4
    flat = np.zeros(max(o, 4), dtype=np.int32)
    for p, off in zip(parts, offs):
        flat[off:off + p.size] = p
    host = torch.from_numpy(flat)
    if device.type == "cuda":
        host = host.pin_memory()
        dev = host.to(device, non_blocking=True)
    else:
        dev = host
    views = [dev[off:off + s] for off, s in zip(offs, sizes)]
    tables = [views[7 + i].view(B, tables_np[i].shape[1]) for i in range(len(tables_np))]
    return StepBatch(n_tokens=T, n_seqs=B, tok_ids=views[0], tok_pos=views[1], tok_seq=views[2],
                     seq_start=views[3], seq_before=views[4], seq_slot=views[5], want_rows=views[6],
                     tables=tables, max_new=int(lens.max()) if B else 0,
                     max_after=int((lens + before).max()) if B else 0,
                     host={"lens": lens, "before": before, "pinned": host})
