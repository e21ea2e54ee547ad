"""A step's batch, as the kernels see it.

The host packs the rows of all sequences of a step one after another and
describes them with a few int32 arrays in ONE buffer, uploaded with one copy:

  tokens[r]     token id of row r
  row_seq[r]    which sequence of this step row r belongs to (0..n_seqs-1)
  row_pos[r]    the row's position in its sequence (tokens already cached + offset)
  seq_starts[s] first row of sequence s (n_seqs + 1 entries)
  kv_lens[s]    length of sequence s after this step
  seq_slots[s]  cache slot of sequence s (indexes fixed-size state)
  want_rows[i]  rows whose logits are asked for
  tables[g]     page ids of each sequence in key/value group g, [n_seqs_cap, table_width]

Building the arrays is plain Python over lists (tested without a GPU); the
device side is one int32 tensor cut into views at fixed offsets, so that a
captured CUDA graph keeps reading the same addresses step after step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np


@dataclass(frozen=True)
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()        # offsets into `tokens` whose logits are wanted


@dataclass
class HostBatch:
    """The packed arrays of one step (NumPy int32), before upload."""
    n_rows: int
    n_seqs: int
    tokens: np.ndarray
    row_seq: np.ndarray
    row_pos: np.ndarray
    seq_starts: np.ndarray
    kv_lens: np.ndarray
    seq_slots: np.ndarray
    want_rows: np.ndarray
    first_pos: list[int]
    max_new: int
    max_kv_len: int

    @property
    def is_decode(self) -> bool:
        return self.max_new == 1


def pack(entries: Sequence[StepEntry], first_positions: Sequence[int], vocab_size: int) -> HostBatch:
    """Packs a step.  `first_positions[i]` is how many tokens sequence i already holds."""
    if not entries:
        raise ValueError("a step needs at least one sequence")
    if len({e.slot for e in entries}) != len(entries):
        raise ValueError("a sequence may appear only once in a step")
    tokens, row_seq, row_pos, want_rows = [], [], [], []
    seq_starts, kv_lens, seq_slots = [0], [], []
    for s, (e, p0) in enumerate(zip(entries, first_positions)):
        n = len(e.tokens)
        if n == 0:
            raise ValueError("a sequence in a step brings at least one token")
        for t in e.tokens:
            if not (0 <= int(t) < vocab_size):
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab_size}")
        base = seq_starts[-1]
        tokens.extend(int(t) for t in e.tokens)
        row_seq.extend([s] * n)
        row_pos.extend(range(p0, p0 + n))
        for w in e.want:
            if not (0 <= int(w) < n):
                raise ValueError(f"wanted place {w} is outside the {n} tokens this step brings")
            want_rows.append(base + int(w))
        seq_starts.append(base + n)
        kv_lens.append(p0 + n)
        seq_slots.append(e.slot)
    i32 = np.int32
    return HostBatch(
        n_rows=len(tokens), n_seqs=len(entries),
        tokens=np.asarray(tokens, i32), row_seq=np.asarray(row_seq, i32), row_pos=np.asarray(row_pos, i32),
        seq_starts=np.asarray(seq_starts, i32), kv_lens=np.asarray(kv_lens, i32),
        seq_slots=np.asarray(seq_slots, i32), want_rows=np.asarray(want_rows, i32),
        first_pos=list(first_positions), max_new=max(len(e.tokens) for e in entries), max_kv_len=max(kv_lens))


class MetaLayout:
    """Offsets of the sections inside the one int32 buffer, for given capacities."""

    def __init__(self, rows_cap: int, seqs_cap: int, table_widths: dict[int, int]):
        self.rows_cap, self.seqs_cap = rows_cap, seqs_cap
        self.table_widths = dict(table_widths)
        off = 0

        def section(n):
            nonlocal off
            start = off
            off += (n + 3) // 4 * 4          # 16-byte aligned sections
            return start

        self.tokens = section(rows_cap)
        self.row_seq = section(rows_cap)
        self.row_pos = section(rows_cap)
        self.seq_starts = section(seqs_cap + 1)
        self.kv_lens = section(seqs_cap)
        self.seq_slots = section(seqs_cap)
        self.want_rows = section(rows_cap)
        self.tables = {g: section(seqs_cap * w) for g, w in self.table_widths.items()}
        self.total = off

    def fill(self, host: np.ndarray, b: HostBatch, tables: dict[int, list[list[int]]]) -> None:
        """Writes a packed step into a host buffer of `total` int32."""
        if b.n_rows > self.rows_cap or b.n_seqs > self.seqs_cap:
            raise ValueError("step exceeds the capacity of its metadata buffer")
        host[self.tokens:self.tokens + b.n_rows] = b.tokens
        host[self.row_seq:self.row_seq + b.n_rows] = b.row_seq
        host[self.row_pos:self.row_pos + b.n_rows] = b.row_pos
        host[self.seq_starts:self.seq_starts + b.n_seqs + 1] = b.seq_starts
        host[self.kv_lens:self.kv_lens + b.n_seqs] = b.kv_lens
        host[self.seq_slots:self.seq_slots + b.n_seqs] = b.seq_slots
        host[self.want_rows:self.want_rows + len(b.want_rows)] = b.want_rows
        for g, w in self.table_widths.items():
            base = self.tables[g]
            for s, pages in enumerate(tables[g]):
                n = min(len(pages), w)
                host[base + s * w: base + s * w + n] = pages[:n]
