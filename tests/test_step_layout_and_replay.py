"""Host-side pieces of a step, without a GPU: the record a step's kernels read (ids, positions,
sequence of each token, first rows, tables; every part on a 16-byte boundary of one buffer) and
the replay loop's decisions (a slot a request, opened at its first step and given back at its end,
a file only where logits are wanted, one line a step)."""
import json
import os

import numpy as np
import pytest
import torch

from ultima_b200.engine.batch import DecodeRecord, build_step_batch
from ultima_b200.engine.trace import replay


def _tables(B, widths, seed=0):
    g = np.random.default_rng(seed)
    return [g.integers(0, 50, size=(B, w)).astype(np.int32) for w in widths]


def test_record_of_a_ragged_step():
    slots = [4, 0, 7]
    new = [[11, 12, 13, 14, 15], [21], [31, 32, 33]]
    before = [0, 70, 3]
    want = [0, 4, 5, 8]
    tables = _tables(3, [3, 2])
    b = build_step_batch(slots, new, before, want, tables, torch.device("cpu"))
    assert (b.n_tokens, b.n_seqs, b.max_new, b.max_after) == (9, 3, 5, 71)
    assert b.tok_ids.tolist() == [11, 12, 13, 14, 15, 21, 31, 32, 33]
    assert b.tok_seq.tolist() == [0, 0, 0, 0, 0, 1, 2, 2, 2]
    assert b.tok_pos.tolist() == [0, 1, 2, 3, 4, 70, 3, 4, 5]          # absolute positions: before + place
    assert b.seq_start.tolist() == [0, 5, 6, 9]
    assert b.seq_before.tolist() == before and b.seq_slot.tolist() == slots
    assert b.want_rows.tolist() == want
    for t, ref in zip(b.tables, tables):
        assert t.shape == ref.shape and np.array_equal(t.numpy(), ref)
    # one buffer, every part at a multiple of four 32-bit words (vector loads, bulk copies)
    base = b.tok_ids.data_ptr()
    for part in [b.tok_ids, b.tok_pos, b.tok_seq, b.seq_start, b.seq_before, b.seq_slot, b.want_rows] + b.tables:
        assert part.dtype == torch.int32 and (part.data_ptr() - base) % 16 == 0
    assert b.host["n_ints"] * 4 >= b.tables[-1].data_ptr() + b.tables[-1].numel() * 4 - base


def test_record_of_one_token_each_and_of_nothing_wanted():
    b = build_step_batch([2, 5], [[9], [8]], [63, 64], [], _tables(2, [4]), torch.device("cpu"))
    assert b.tok_pos.tolist() == [63, 64] and b.tok_seq.tolist() == [0, 1] and b.seq_start.tolist() == [0, 1, 2]
    assert b.want_rows.numel() == 0 and b.max_new == 1 and b.max_after == 65


def test_decode_record_keeps_its_layout_from_step_to_step():
    """The record of a captured decode step: the same places as ``build_step_batch`` makes for one
    token a sequence with every logit wanted, so a graph that was captured on it reads the right
    words after every update."""
    B, widths = 3, [2, 5]
    slots, before = [6, 1, 3], [10, 64, 127]
    tables = _tables(B, widths, seed=3)
    ref = build_step_batch(slots, [[5], [6], [7]], before, [0, 1, 2], tables, torch.device("cpu"))

    class Ring:                                           # stands in for the pinned buffers
        def take(self, n):
            return 0, torch.zeros(n, dtype=torch.int32)

        def copied(self, i):
            pass
    rec = DecodeRecord(B, widths, torch.device("cpu"), Ring())
    got = rec.update(slots, [5, 6, 7], before, tables)
    for name in ("tok_ids", "tok_pos", "tok_seq", "seq_start", "seq_before", "seq_slot", "want_rows"):
        assert getattr(got, name).tolist() == getattr(ref, name).tolist(), name
    for t, r in zip(got.tables, ref.tables):
        assert torch.equal(t, r)
    assert got.max_after == 128 and got.max_new == 1
    # the next step: same tensors (a graph holds their addresses), new contents
    again = rec.update(slots, [1, 2, 3], [11, 65, 128], tables)
    assert again.tok_ids.data_ptr() == got.tok_ids.data_ptr() and again.tok_ids.tolist() == [1, 2, 3]
    assert again.tok_pos.tolist() == [11, 65, 128] and again.max_after == 129


class ReplayEngine:
    """Logits are stand-ins: the row for a wanted place holds (slot, absolute position, token)."""

    def __init__(self, n_slots=3):
        self.free = list(range(n_slots))[::-1]
        self.held = {}
        self.steps, self.closed = [], []

    def open(self, n):
        assert n <= len(self.free), "more live requests than slots"
        got = [self.free.pop() for _ in range(n)]
        for s in got:
            self.held[s] = 0
        return got

    def close(self, slots):
        for s in slots:
            assert s in self.held, "slot given back twice"
            del self.held[s]
            self.free.append(s)
            self.closed.append(s)

    def step(self, slots, tokens, want):
        rows = []
        for s, t, w in zip(slots, tokens, want):
            assert s in self.held
            rows += [[s, self.held[s] + p, t[p]] for p in w]
            self.held[s] += len(t)
        self.steps.append((list(slots), [list(t) for t in tokens]))
        return torch.tensor(rows, dtype=torch.float32).reshape(len(rows), 3)

    def check_errors(self):
        pass


def test_replay_opens_a_slot_a_request_and_gives_it_back_at_its_end(tmp_path):
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]},
                                {"id": "b", "tokens": [9], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}, {"id": "b", "tokens": [8], "want": [0]}],
         "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [6], "want": []}], "end": ["a", "never seen"]},
        # a second batch: its requests take the slots that came back
        {"step": 7, "entries": [{"id": "c", "tokens": [1, 2], "want": [1]}, {"id": "b", "tokens": [3], "want": [0]},
                                {"id": "d", "tokens": [4, 4, 4], "want": []}], "end": ["c", "b", "d"]},
    ]
    eng = ReplayEngine(n_slots=3)
    said = []
    n = replay(eng, [json.dumps(x) for x in lines] + ["", "  "], str(tmp_path), said.append)
    assert n == 4 and said == ["done 0", "done 1", "done 2", "done 7"]
    assert not eng.held and sorted(eng.free) == [0, 1, 2] and len(eng.closed) == 5
    # a request keeps its slot from step to step
    a_slot = eng.steps[0][0][0]
    assert eng.steps[1][0][0] == a_slot and eng.steps[2][0] == [a_slot]
    # files only where something was wanted, rows in the order of the entries and of ``want``
    assert sorted(os.listdir(tmp_path)) == ["0.f32", "1.f32", "7.f32"]
    f0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(-1, 3)
    assert f0.tolist() == [[a_slot, 0, 5], [a_slot, 2, 3]]
    f1 = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(-1, 3)
    b_slot = eng.steps[0][0][1]
    assert f1.tolist() == [[a_slot, 3, 4], [b_slot, 1, 8]]
    f7 = np.fromfile(tmp_path / "7.f32", dtype="<f4").reshape(-1, 3)
    assert [r[1:] for r in f7.tolist()] == [[1, 2], [0, 3]]             # "b" of the second batch starts at 0 again


def test_replay_stops_at_a_line_that_is_no_json(tmp_path):
    eng = ReplayEngine()
    with pytest.raises(json.JSONDecodeError):
        replay(eng, ['{"step": 0, "entries": [], "end": []}', "not json"], str(tmp_path), None)
