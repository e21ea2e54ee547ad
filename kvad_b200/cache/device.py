"""Device storage of the cache.

For every key/value group: two tensors `[layers of the group, pages,
kv heads, 64, head size]` in the engine's dtype.  A page of one head is one
contiguous tile, which is what the attention kernels read.  For every state
group: `[layers of the group, slots, *shape]`, zeroed when a slot is handed
out (bisand/kvad zeroes `CacheShape.state` the same way,
crates/llm/src/model/mod.rs:636-646, 732-736).  Which page belongs to which
sequence is the host's knowledge (`SlotBook`); each step uploads the page
lists of the sequences it runs.

Sized once, from a token budget: `max_tokens` live tokens, each sequence
rounded up to whole pages.  A freed slot's pages are reused as they are;
nothing is cleared, because a sequence never reads past its own length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .layout import CacheLayout, KVNeed, StateNeed
from .pages import PAGE_SIZE, SlotBook


@dataclass
class KVView:
    """One cache entry's pages as a mixer sees them during a step."""
    k_pages: torch.Tensor          # [pages, kv heads, page size, head size]
    v_pages: torch.Tensor
    page_table: torch.Tensor       # int32 [sequences of the step, table width], this group's
    window: Optional[int]
    page_size: int


class DeviceCache:
    def __init__(self, layout: CacheLayout, dtype: torch.dtype, device, max_tokens: int, *,
                 max_seqs: Optional[int] = None, max_positions: Optional[int] = None,
                 page_size: int = PAGE_SIZE):
        self.layout = layout
        self.dtype = dtype
        self.device = torch.device(device)
        self.page_size = page_size
        self.max_positions = max_positions
        n_pages = max(1, -(-int(max_tokens) // page_size))
        self.n_pages = n_pages
        self.max_tokens = n_pages * page_size
        self.n_slots = int(max_seqs) if max_seqs else min(n_pages, 4096)
        per_seq = max_positions if max_positions else self.max_tokens
        self.table_width = max(1, -(-per_seq // page_size))

        self.kv: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        self.state: dict[int, torch.Tensor] = {}
        pages_per_group, windows = [], []
        self._kv_group_index: dict[int, int] = {}     # layout group -> index among kv groups (SlotBook's numbering)
        for g, group in enumerate(layout.groups):
            need = group.need
            if isinstance(need, KVNeed):
                shape = (len(group.entries), n_pages, need.n_kv_heads, page_size, need.head_dim)
                self.kv[g] = (torch.empty(shape, dtype=dtype, device=self.device),
                              torch.empty(shape, dtype=dtype, device=self.device))
                self._kv_group_index[g] = len(pages_per_group)
                pages_per_group.append(n_pages)
                windows.append(need.window)
            elif isinstance(need, StateNeed):
                self.state[g] = torch.zeros((len(group.entries), self.n_slots, *need.shape),
                                            dtype=need.dtype, device=self.device)
        self.book = SlotBook(self.n_slots, pages_per_group, windows, page_size, max_positions)

    # -- slots -------------------------------------------------------------------
    def acquire(self) -> int:
        slot = self.book.acquire()
        for t in self.state.values():
            t[:, slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.book.release(slot)

    def length(self, slot: int) -> int:
        return self.book.length[slot]

    # -- views ---------------------------------------------------------------------
    def kv_group_ids(self) -> list[int]:
        return list(self.kv)

    def pages_of(self, slot: int, group: int) -> list[int]:
        return self.book.pages[slot][self._kv_group_index[group]]

    def kv_view(self, entry: int, page_tables: dict[int, torch.Tensor]) -> KVView:
        g, i = self.layout.place(entry)
        k, v = self.kv[g]
        need = self.layout.groups[g].need
        return KVView(k[i], v[i], page_tables[g], need.window, self.page_size)

    def state_view(self, entry: int) -> torch.Tensor:
        """`[slots, *shape]` of one entry; rows are indexed by slot id."""
        g, i = self.layout.place(entry)
        return self.state[g][i]

    # -- accounting ----------------------------------------------------------------
    def bytes(self) -> int:
        n = 0
        for k, v in self.kv.values():
            n += k.numel() * k.element_size() * 2
        for s in self.state.values():
            n += s.numel() * s.element_size()
        return n
