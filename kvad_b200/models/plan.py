"""A model as data, and the object built from it.

`ModelPlan` is what an architecture makes of its configuration: the
embedding, one `PartSpec` per block (so layers may differ in mixer and
feed-forward), the head, and the ORDER in which blocks run.  The order is a
list of `LayerCall(layer, cache, writes_cache)`: a block may be named twice
(its weights run twice, each call with a cache entry of its own), and a call
may read the cache entry another call writes.  `Model` builds the parts from
the plan through the part registries, collects their tensor requests for the
audit, loads them, and runs a step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..cache.layout import CacheLayout
from ..parts.base import PartSpec, build_part
from ..weights.source import TensorRequest, WeightSource


@dataclass(frozen=True)
class LayerCall:
    layer: int                 # which block's weights
    cache: int                 # which cache entry its mixer uses
    writes_cache: bool = True  # False: reads what another call wrote to that entry


@dataclass(frozen=True)
class ModelPlan:
    arch_id: str
    vocab_size: int
    width: int
    embedding: PartSpec
    blocks: tuple[PartSpec, ...]                  # family "block"; params carry the inner PartSpecs
    block_prefixes: tuple[str, ...]
    head: PartSpec
    order: tuple[LayerCall, ...]
    ignored_suffixes: tuple[str, ...] = ()        # buffers in checkpoints that are not weights
    eos_token_ids: tuple[int, ...] = ()
    summary: str = ""
    #: the longest sequence the model takes, whatever bounds it (a learned position table, the range a
    #: rotary encoding was trained for, a configuration key); None: only the cache bounds a sequence.
    #: A position table in the embedding bounds it too; the smaller of the two holds.
    max_positions: Optional[int] = None

    @staticmethod
    def straight_order(n_layers: int) -> tuple[LayerCall, ...]:
        return tuple(LayerCall(i, i) for i in range(n_layers))


class Model:
    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding, "")
        self.blocks = [build_part("block", spec, prefix) for spec, prefix in zip(plan.blocks, plan.block_prefixes)]
        self.head = build_part("head", plan.head, "", embedding=self.embedding)
        for call in plan.order:
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"the run order names block {call.layer}, the model has {len(self.blocks)}")
        self.cache_layout = self._cache_layout()
        self.dtype: Optional[torch.dtype] = None
        self.device = None

    # -- cache needs -------------------------------------------------------------
    def _cache_layout(self) -> CacheLayout:
        n_entries = 1 + max((c.cache for c in self.plan.order), default=-1)
        needs: list = [None] * n_entries
        written = [False] * n_entries
        for call in self.plan.order:
            need = self.blocks[call.layer].mixer.cache_need()
            if needs[call.cache] is not None and needs[call.cache] != need:
                raise ValueError(f"cache entry {call.cache} is used by mixers with different needs")
            needs[call.cache] = need
            if call.writes_cache:
                if written[call.cache]:
                    raise ValueError(f"cache entry {call.cache} is written by two calls of the run order")
                written[call.cache] = True
            elif not written[call.cache]:
                raise ValueError(f"a call reads cache entry {call.cache} before any call has written it")
        return CacheLayout(needs)

    @property
    def max_positions(self) -> Optional[int]:
        """The longest sequence: the plan's own bound and the embedding's position table, whichever is smaller."""
        bounds = [b for b in (self.plan.max_positions, getattr(self.embedding, "max_positions", None)) if b]
        return min(bounds) if bounds else None

    @property
    def graph_safe(self) -> bool:
        """Whether every part's launches depend on a step's shape only (see `Part.graph_safe`)."""
        return all(p.all_graph_safe() for p in self.parts())

    # -- weights -------------------------------------------------------------------
    def parts(self):
        return [self.embedding, *self.blocks, self.head]

    def requests(self) -> list[TensorRequest]:
        out: list[TensorRequest] = []
        for p in self.parts():
            out.extend(p.requests())
        return out

    def load(self, source: WeightSource, dtype: torch.dtype, device) -> "Model":
        for name in getattr(self.head, "skipped", []):
            source.skip(name)
        source.check(self.requests())

        def fetch(name, transpose=False, keep_f32=False, optional=False):
            if optional and not source.has(name):
                return None
            return source.fetch(name, compute_dtype=dtype, device=device, transpose=transpose, keep_f32=keep_f32)

        for p in self.parts():
            p.load(fetch)
        self.dtype, self.device = dtype, torch.device(device)
        return self

    def tensors(self) -> list[torch.Tensor]:
        seen, out = set(), []
        for p in self.parts():
            for t in p.tensors():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    out.append(t)
        return out

    def param_count(self) -> int:
        return sum(t.numel() for t in self.tensors())

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())

    # -- one step --------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Runs the step's rows through the model; returns float32 logits of the wanted rows."""
        ctx.ops.begin_step()
        x = self.embedding.forward(ctx)
        for call in self.plan.order:
            self.blocks[call.layer].forward(ctx, x, call)
        logits = self.head.forward(ctx, x)
        ctx.ops.end_step()
        return logits
