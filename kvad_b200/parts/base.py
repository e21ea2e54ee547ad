"""The parts a model is put together from, and where they are registered.

Five families: position encodings, norms, mixers, feed-forwards, and block
arrangements (plus the two ends of a model, the token embedding and the output
head).  A part is a class that takes its sizes and constants as constructor
parameters, says which tensors it needs from a checkpoint, loads them, and
runs on a step's rows.  No part knows which model it is in: an architecture
describes itself as data (`PartSpec(kind, params)` per part, layer by layer)
and the parts are looked up here by family and kind.  Registering a new kind
takes one call and no change to this package.

Interfaces (all rows of a step are packed; `ctx` is the step's `StepContext`):

* `Norm.forward(ctx, x, rows=None) -> Tensor`: normalises rows of the
  float32 residual stream `x` (only the listed rows if `rows` is given) into
  a new buffer of the compute dtype.
* `PositionEncoding.table() -> Tensor | None`: a table `[positions, width]`
  that the token embedding adds per row, or None; `rotate(ctx, q, k)`: in
  place change of a mixer's queries and keys by the rows' positions (identity
  for encodings that act at the embedding); `max_positions`: the bound it
  puts on a sequence's length, or None.
* `Mixer.cache_need() -> KVNeed | StateNeed | None`;
  `Mixer.forward(ctx, h, residual, call)`: reads normalised rows `h`, mixes
  information between positions of a sequence through the cache entry
  `call.cache`, and ADDS its output to `residual` (float32) in place.
* `FeedForward.forward(ctx, h, residual)`: position-wise; adds to `residual`.
* `Block.forward(ctx, x, call)`: one layer on the residual stream `x`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Optional

import torch

from ..weights.source import TensorRequest

FAMILIES = ("position", "norm", "mixer", "feed_forward", "block", "embedding", "head")
_PARTS: dict[str, dict[str, type]] = {f: {} for f in FAMILIES}


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more) -> "PartSpec":
        return PartSpec(self.kind, {**self.params, **more})


def register_part(family: str, kind: str, cls: type, *, replace: bool = False) -> type:
    if family not in _PARTS:
        raise ValueError(f"unknown family `{family}`; families are {FAMILIES}")
    if kind in _PARTS[family] and not replace:
        raise ValueError(f"{family} `{kind}` is already registered")
    _PARTS[family][kind] = cls
    return cls


def unregister_part(family: str, kind: str) -> None:
    _PARTS[family].pop(kind, None)


def part_kinds(family: str) -> list[str]:
    return sorted(_PARTS[family])


def build_part(family: str, spec: PartSpec, prefix: str = "", **extra):
    try:
        cls = _PARTS[family][spec.kind]
    except KeyError:
        raise ValueError(f"no {family} of kind `{spec.kind}`; registered: {part_kinds(family)}") from None
    return cls(prefix=prefix, **dict(spec.params), **extra)


Fetch = Callable[..., torch.Tensor]   # fetch(name, transpose=False, keep_f32=False) -> device tensor


class Part:
    """Base of all parts: tensor requests, loading, accounting."""

    #: True if what the part launches for a step depends only on the step's SHAPE (rows, sequences,
    #: longest run of new rows, wanted rows) and on device memory - never on host-side values such as
    #: positions, lengths or slot ids.  Steps of a model whose parts all say so are captured as CUDA
    #: graphs and replayed.  A part that loops over host data leaves this False and runs kernel by kernel.
    graph_safe = False

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def all_graph_safe(self) -> bool:
        return bool(self.graph_safe) and all(c.all_graph_safe() for c in self.children())

    def children(self) -> list["Part"]:
        return []

    def own_requests(self) -> list[TensorRequest]:
        return []

    def requests(self) -> list[TensorRequest]:
        out = list(self.own_requests())
        for c in self.children():
            out.extend(c.requests())
        return out

    def load_own(self, fetch: Fetch) -> None:
        pass

    def load(self, fetch: Fetch) -> None:
        self.load_own(fetch)
        for c in self.children():
            c.load(fetch)

    def own_tensors(self) -> list[torch.Tensor]:
        return []

    def tensors(self) -> list[torch.Tensor]:
        out = list(self.own_tensors())
        for c in self.children():
            out.extend(c.tensors())
        return out


class PositionEncoding(Part):
    max_positions: Optional[int] = None

    def table(self) -> Optional[torch.Tensor]:
        return None

    def rotate(self, ctx, q: torch.Tensor, k: torch.Tensor) -> None:
        return None


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, call) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, ctx, x: torch.Tensor, call) -> None:
        raise NotImplementedError
