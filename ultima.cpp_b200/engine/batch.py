"""One step's worth of tokens, laid out for the kernels.

A step brings, for each of its sequences, some new tokens that follow what the sequence's
slot already holds.  Tokens of all sequences are packed one after another; for every token
the kernels get its id, its absolute position and the index of its sequence in the step,
and for every sequence its first row, its length before the step and its slot.  All of it
is one int32 record, written into pinned host memory and moved to the device in one copy.
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


class PinnedRing:
    """A few pinned host buffers used in turn for the step records.  A buffer is written again
    only after the copy that last read it has finished (an event recorded behind that copy)."""

    def __init__(self, device, n_buffers: int = 4, n_ints: int = 1 << 14):
        self.device = device
        self.n = n_buffers
        self.size = n_ints
        self.bufs = [None] * n_buffers
        self.events = [None] * n_buffers
        self.next = 0

    def take(self, n_ints: int):
        i = self.next
        self.next = (i + 1) % self.n
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i] is None or self.bufs[i].numel() < n_ints:
            size = max(self.size, 1 << (max(n_ints, 1) - 1).bit_length())
            self.bufs[i] = torch.empty(size, dtype=torch.int32).pin_memory()
        return i, self.bufs[i]

    def copied(self, i: int) -> None:
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


def build_step_batch(slots, new_tokens, before, want_rows, tables_np, device, ring: PinnedRing | None = None,
                     static: torch.Tensor | None = None) -> StepBatch:
    """slots: slot of each sequence; new_tokens: list of int sequences; before: positions
    already held; want_rows: rows (in the packed order) whose logits are wanted;
    tables_np: per KV group an int32 array [B, pages].  ``static``: a device buffer to fill
    instead of a fresh one (the same layout step after step, for a captured graph)."""
    B = len(slots)
    lens = np.fromiter((len(t) for t in new_tokens), dtype=np.int64, count=B)
    T = int(lens.sum())
    start = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(lens, out=start[1:])
    if T == B:                      # one token a sequence
        ids = np.fromiter((t[0] for t in new_tokens), dtype=np.int32, count=B)
        seq = np.arange(B, dtype=np.int32)
    else:
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
    total = max(o, 4)
    if device.type == "cuda":
        if ring is None:
            ring = PinnedRing(device, 1, total)
        idx, host = ring.take(total)
        flat = host.numpy()
        for p, off in zip(parts, offs):
            flat[off:off + p.size] = p
        if static is not None:
            if static.numel() < total:
                raise ValueError("static step record is too small")
            dev = static
            dev[:total].copy_(host[:total], non_blocking=True)
        else:
            dev = host[:total].to(device, non_blocking=True)
        ring.copied(idx)
    else:
        flat = np.zeros(total, dtype=np.int32)
        for p, off in zip(parts, offs):
            flat[off:off + p.size] = p
        dev = torch.from_numpy(flat)
    views = [dev[off:off + s] for off, s in zip(offs, sizes)]
    tables = [views[7 + i].view(B, tables_np[i].shape[1]) for i in range(len(tables_np))]
    return StepBatch(n_tokens=T, n_seqs=B, tok_ids=views[0], tok_pos=views[1], tok_seq=views[2],
                     seq_start=views[3], seq_before=views[4], seq_slot=views[5], want_rows=views[6],
                     tables=tables, max_new=int(lens.max()) if B else 0,
                     max_after=int((lens + before).max()) if B else 0,
                     host={"lens": lens, "before": before, "n_ints": total})


class DecodeRecord:
    """The step record of a decode step of ``B`` sequences (one token each, every logit wanted), laid
    out once: the same parts in the same places as ``build_step_batch`` makes, in one device buffer
    that a captured graph reads.  From step to step only the token ids, the positions, the lengths
    before the step and (at page edges) the tables change."""

    def __init__(self, B: int, table_widths: list, device, ring: PinnedRing):
        self.B, self.device, self.ring = B, device, ring
        sizes = [B, B, B, B + 1, B, B, B] + [B * w for w in table_widths]
        self.offs, o = [], 0
        for n in sizes:
            self.offs.append(o)
            o += -(-n // 4) * 4
        self.total = max(o, 4)
        self.sizes, self.table_widths = sizes, list(table_widths)
        self.host = np.zeros(self.total, dtype=np.int32)
        ar = np.arange(B + 1, dtype=np.int32)
        self.host[self.offs[2]:self.offs[2] + B] = ar[:B]            # sequence of each token
        self.host[self.offs[3]:self.offs[3] + B + 1] = ar             # first row of each sequence
        self.host[self.offs[6]:self.offs[6] + B] = ar[:B]            # every row is wanted
        self.static = torch.zeros(self.total, dtype=torch.int32, device=device)
        v = [self.static[off:off + n] for off, n in zip(self.offs, sizes)]
        tables = [v[7 + i].view(B, w) for i, w in enumerate(table_widths)]
        self.batch = StepBatch(n_tokens=B, n_seqs=B, tok_ids=v[0], tok_pos=v[1], tok_seq=v[2], seq_start=v[3],
                               seq_before=v[4], seq_slot=v[5], want_rows=v[6], tables=tables, max_new=1,
                               max_after=0, host={"n_ints": self.total})

    def update(self, slots, ids, before, tables_np, ids_dev=None) -> StepBatch:
        """``ids_dev`` (int32 on the device, one a sequence) instead of ``ids``: the token ids are copied
        from there on the device, and the host's copy leaves that part of the record alone."""
        h, o, B = self.host, self.offs, self.B
        if ids_dev is None:
            h[o[0]:o[0] + B] = ids
        h[o[1]:o[1] + B] = before
        h[o[4]:o[4] + B] = before
        h[o[5]:o[5] + B] = slots
        for i, t in enumerate(tables_np):
            h[o[7 + i]:o[7 + i] + t.size] = t.reshape(-1)
        idx, pinned = self.ring.take(self.total)
        pinned.numpy()[:self.total] = h
        if ids_dev is None:
            self.static.copy_(pinned[:self.total], non_blocking=True)
        else:
            self.static[o[1]:].copy_(pinned[o[1]:self.total], non_blocking=True)
            self.static[:B].copy_(ids_dev[:B], non_blocking=True)
        self.ring.copied(idx)
        b = self.batch
        b.max_after = int(max(before)) + 1
        b.host["lens"] = np.ones(B, dtype=np.int64)
        b.host["before"] = np.asarray(before, dtype=np.int32)
        return b
