"""Host-side bookkeeping of the cache: slots, pages and lengths.

Pure Python and free of CUDA, so that its invariants are tested on any
machine: a slot or a page is never handed out twice, never freed twice, and
every one of them is back in its pool when all sequences have ended.

A *slot* stands for one live sequence; it owns, for every key/value group, the
pages that hold its positions (64 positions a page), and its length.  A group
that keeps only a window drops the pages that have slid out of every later
query's reach.  The cache's capacity is a number of pages per group, i.e. a
number of tokens rounded up per sequence to whole pages.
"""
from __future__ import annotations

from typing import Optional, Sequence

PAGE_SIZE = 64


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    pass


class IdPool:
    """Hands out integers 0..n-1; remembers which are out."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free = list(range(self.n - 1, -1, -1))   # pop() gives the lowest id first
        self._out: set[int] = set()

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are in use)")
        i = self._free.pop()
        self._out.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._out:
            raise CacheError(f"{self.what} {i} was given back but is not in use")
        self._out.remove(i)
        self._free.append(i)

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_out(self) -> int:
        return len(self._out)

    def is_out(self, i: int) -> bool:
        return i in self._out


class SlotBook:
    """Slots, their lengths, and their pages in every key/value group."""

    def __init__(self, n_slots: int, pages_per_group: Sequence[int], windows: Sequence[Optional[int]],
                 page_size: int = PAGE_SIZE, max_positions: Optional[int] = None):
        if len(pages_per_group) != len(windows):
            raise ValueError("one window entry (or None) per group")
        self.page_size = int(page_size)
        self.max_positions = max_positions
        self.slots = IdPool(n_slots, "slot")
        self.pools = [IdPool(n, f"page of group {g}") for g, n in enumerate(pages_per_group)]
        self.windows = list(windows)
        self.length: dict[int, int] = {}
        # pages[slot][group] = list over page index (position // page_size) of page id, or -1 once dropped
        self.pages: dict[int, list[list[int]]] = {}

    # -- slots -------------------------------------------------------------------
    def acquire(self) -> int:
        s = self.slots.take()
        self.length[s] = 0
        self.pages[s] = [[] for _ in self.pools]
        return s

    def release(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheError(f"slot {slot} was released but is not in use")
        for g, table in enumerate(self.pages[slot]):
            for p in table:
                if p >= 0:
                    self.pools[g].give_back(p)
        del self.pages[slot]
        del self.length[slot]
        self.slots.give_back(slot)

    def live_slots(self) -> list[int]:
        return sorted(self.length)

    # -- growth ------------------------------------------------------------------
    def pages_needed(self, slot: int, new_tokens: int) -> list[int]:
        """How many new pages each group must hand out for `new_tokens` more positions."""
        new_len = self.length[slot] + new_tokens
        want = -(-new_len // self.page_size)
        return [max(0, want - len(table)) for table in self.pages[slot]]

    def grow(self, slot: int, new_tokens: int) -> int:
        """Makes room for `new_tokens` more positions; returns the position of the first.

        Either every group gets its pages or nothing changes."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not in use")
        if new_tokens <= 0:
            raise CacheError("a step brings at least one token per sequence")
        first = self.length[slot]
        new_len = first + new_tokens
        if self.max_positions is not None and new_len > self.max_positions:
            raise CacheError(f"context window of {self.max_positions} tokens is full")
        need = self.pages_needed(slot, new_tokens)
        for g, n in enumerate(need):
            if n > self.pools[g].n_free:
                raise CacheFull(
                    f"the cache is full: group {g} needs {n} more page(s) of {self.page_size} tokens, "
                    f"{self.pools[g].n_free} of {self.pools[g].n} are free")
        for g, n in enumerate(need):
            for _ in range(n):
                self.pages[slot][g].append(self.pools[g].take())
        self.length[slot] = new_len
        return first

    def trim_windows(self, slot: int) -> None:
        """Drops pages that no later query of a windowed group can reach."""
        n = self.length[slot]
        for g, w in enumerate(self.windows):
            if w is None:
                continue
            first_needed = max(0, n - w + 1)     # the next query sits at position n
            table = self.pages[slot][g]
            for i in range(min(len(table), first_needed // self.page_size)):
                if table[i] >= 0:
                    self.pools[g].give_back(table[i])
                    table[i] = -1

    def truncate(self, slot: int, length: int) -> int:
        """Rewinds a sequence to `length` positions; returns where it landed.

        Pages past the new end go back; a windowed group cannot bring dropped
        pages back, so a rewind into them is refused."""
        cur = self.length[slot]
        length = max(0, min(length, cur))
        for g, table in enumerate(self.pages[slot]):
            keep = -(-length // self.page_size)
            if self.windows[g] is not None and any(p < 0 for p in table[:keep]) and length < cur:
                first_needed = max(0, length - self.windows[g] + 1)
                if any(p < 0 for p in table[first_needed // self.page_size:keep]):
                    raise CacheError("cannot rewind into positions a windowed group has already dropped")
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    self.pools[g].give_back(p)
        self.length[slot] = length
        return length

    # -- accounting ----------------------------------------------------------------
    def tokens_held(self) -> int:
        """Live tokens, each sequence rounded up to whole pages."""
        return sum(-(-n // self.page_size) * self.page_size for n in self.length.values())

    def check_all_free(self) -> None:
        if self.slots.n_out or any(p.n_out for p in self.pools):
            raise CacheError(f"leak: {self.slots.n_out} slot(s) and {[p.n_out for p in self.pools]} page(s) still out")
