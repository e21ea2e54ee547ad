"""What a part sees of a step: the rows' metadata on the device, scratch
buffers, the cache, and the kernels.

Scratch comes from an arena: one device allocation, handed out front to back
and reset at the start of every step.  The same sequence of requests gives the
same addresses, which is what lets a decode step be captured in a CUDA graph
and replayed.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..cache.device import DeviceCache, KVView
from ..ops import Ops
from .batch import HostBatch, MetaLayout


class Arena:
    ALIGN = 1024

    def __init__(self, device, nbytes: int = 0):
        self.device = torch.device(device)
        self.generation = 0
        self._buf = torch.empty(max(nbytes, self.ALIGN), dtype=torch.uint8, device=self.device)
        self._off = 0
        self._high = 0
        self._overflow: list[torch.Tensor] = []

    def reset(self) -> None:
        if self._overflow:
            # the last step needed more than the arena held: grow once, so that later steps fit
            need = self._high + sum(t.numel() for t in self._overflow) + self.ALIGN * (len(self._overflow) + 1)
            self._overflow.clear()
            self._buf = torch.empty(int(need * 1.25), dtype=torch.uint8, device=self.device)
            self.generation += 1
        self._off = 0
        self._high = 0

    def reserve(self, nbytes: int) -> None:
        if nbytes > self._buf.numel():
            self._buf = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
            self.generation += 1

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self._off + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if start + nbytes > self._buf.numel():
            t = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self.device)
            self._overflow.append(t)
            return t[:nbytes].view(dtype).view(*shape)
        self._off = start + nbytes
        self._high = max(self._high, self._off)
        return self._buf[start:start + nbytes].view(dtype).view(*shape)


class DeviceMeta:
    """The device copy of a step's int32 metadata, with pinned host staging."""

    STAGES = 4

    def __init__(self, layout: MetaLayout, device):
        self.layout = layout
        self.device = torch.device(device)
        self.dev = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
        self._host = [torch.zeros(layout.total, dtype=torch.int32).pin_memory() for _ in range(self.STAGES)]
        self._events: list[Optional[torch.cuda.Event]] = [None] * self.STAGES
        self._next = 0
        L = layout
        self.tokens = self.dev[L.tokens:L.tokens + L.rows_cap]
        self.row_seq = self.dev[L.row_seq:L.row_seq + L.rows_cap]
        self.row_pos = self.dev[L.row_pos:L.row_pos + L.rows_cap]
        self.seq_starts = self.dev[L.seq_starts:L.seq_starts + L.seqs_cap + 1]
        self.kv_lens = self.dev[L.kv_lens:L.kv_lens + L.seqs_cap]
        self.seq_slots = self.dev[L.seq_slots:L.seq_slots + L.seqs_cap]
        self.want_rows = self.dev[L.want_rows:L.want_rows + L.rows_cap]
        self.tables = {g: self.dev[off:off + L.seqs_cap * w].view(L.seqs_cap, w)
                       for (g, off), w in zip(L.tables.items(), L.table_widths.values())}

    def upload(self, batch: HostBatch, tables: dict[int, list[list[int]]], *, keep_tokens: bool = False) -> int:
        """Copies a packed step to the device (one asynchronous copy from pinned memory); returns the
        bytes copied.  With `keep_tokens` the token section is left as the device has it: the tokens
        were put there by the sampling of the step before."""
        i = self._next
        self._next = (i + 1) % self.STAGES
        if self._events[i] is not None:
            self._events[i].synchronize()
        host = self._host[i]
        self.layout.fill(host.numpy(), batch, tables)
        start = self.layout.row_seq if keep_tokens else 0
        self.dev[start:].copy_(host[start:], non_blocking=True)
        ev = self._events[i] or torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        return (self.layout.total - start) * 4


class StepContext:
    def __init__(self, ops: Ops, cache: DeviceCache, arena: Arena, meta: DeviceMeta, batch: HostBatch):
        self.ops = ops
        self.dtype = ops.dtype
        self.cache = cache
        self.arena = arena
        self.meta = meta
        self.batch = batch
        self.n_rows = batch.n_rows
        self.n_seqs = batch.n_seqs
        self.n_want = int(len(batch.want_rows))
        self.tokens = meta.tokens
        self.row_seq = meta.row_seq
        self.row_pos = meta.row_pos
        self.seq_starts = meta.seq_starts
        self.kv_lens = meta.kv_lens
        self.seq_slots = meta.seq_slots
        self.want_rows = meta.want_rows
        self.page_tables = meta.tables

    def buffer(self, shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return self.arena.take(shape, dtype or self.dtype)

    def kv(self, entry: int) -> KVView:
        return self.cache.kv_view(entry, self.page_tables)

    def state(self, entry: int) -> torch.Tensor:
        return self.cache.state_view(entry)
