"""What the layers of a model keep per sequence, and how that is grouped.

A mixer declares its need: keys and values per position (`KVNeed`, optionally
only a window of the latest positions) or a block of fixed size per sequence
(`StateNeed`), or nothing.  The model's run order gives every mixer call a
cache entry; entries with the same need form a group, and each group has
storage of its own.  bisand/kvad says the same with `CacheShape{k, v, state}`
per layer and `CacheLayout::per_layer` (crates/llm/src/model/mod.rs:102-220).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch


@dataclass(frozen=True)
class KVNeed:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every position is kept

    def __post_init__(self):
        if self.n_kv_heads <= 0 or self.head_dim <= 0:
            raise ValueError("a key/value cache needs positive head count and head size")
        if self.window is not None and self.window <= 0:
            raise ValueError("a window must be positive")


@dataclass(frozen=True)
class StateNeed:
    shape: tuple[int, ...]           # per sequence
    dtype: torch.dtype = torch.float32


Need = Union[KVNeed, StateNeed, None]


@dataclass(frozen=True)
class Group:
    need: Union[KVNeed, StateNeed]
    entries: tuple[int, ...]         # cache entry ids, in order; index in this tuple = layer index in storage


class CacheLayout:
    """Cache entries (one per mixer call that keeps something) and their groups."""

    def __init__(self, needs: Sequence[Need]):
        self.needs = tuple(needs)
        groups: list[Group] = []
        where: dict[int, tuple[int, int]] = {}
        by_need: dict[object, list[int]] = {}
        for entry, need in enumerate(self.needs):
            if need is None:
                continue
            by_need.setdefault(need, []).append(entry)
        for need, entries in by_need.items():
            g = len(groups)
            groups.append(Group(need, tuple(entries)))
            for i, e in enumerate(entries):
                where[e] = (g, i)
        self.groups = tuple(groups)
        self._where = where

    def place(self, entry: int) -> tuple[int, int]:
        """(group index, index within the group's storage) of a cache entry."""
        return self._where[entry]

    @property
    def kv_groups(self) -> list[int]:
        return [i for i, g in enumerate(self.groups) if isinstance(g.need, KVNeed)]

    @property
    def state_groups(self) -> list[int]:
        return [i for i, g in enumerate(self.groups) if isinstance(g.need, StateNeed)]

    def bytes_per_token(self, element_size: int) -> int:
        """Key and value bytes one position of one sequence takes over all layers."""
        total = 0
        for g in self.groups:
            if isinstance(g.need, KVNeed):
                total += 2 * len(g.entries) * g.need.n_kv_heads * g.need.head_dim * element_size
        return total
